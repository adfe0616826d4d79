"""CPU oracle for the operators next to the mLSTM cell -- TEST INFRASTRUCTURE, NOT PRODUCT.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may import this module.

Restates, with explicit rounding points, what the reference computes eagerly:

* ``add_rmsnorm``: ``x = x + y`` (``xlstm/xlstm_large/model.py:499-510``) followed by ``RMSNorm.forward``
  (``xlstm/xlstm_large/components.py:86-97``: fp32 reduction, result cast to the input dtype, then ``* weight``
  in the input dtype, ``components.py:58-63``);
* ``headnorm_gate``: ``MultiHeadLayerNorm.forward`` on the transposed cell output (``components.py:171-179,
  229-242``: fp32 mean / biased variance, cast, reshape, ``* weight``) and the output gate
  ``sigmoid(o_preact) * h_norm`` (``model.py:445-449``).

* ``soft_cap``: ``cap * tanh(values / cap)`` (``components.py:5-22``), every operator in the input dtype.

Pinning: ``tests/golden/make_golden_layer.py`` ran the reference's own ``RMSNorm`` and ``MultiHeadLayerNorm``
modules and its ``soft_cap`` function in this container and committed inputs and outputs; ``tests/test_oracle_layer_ops.py`` checks this
restatement against them.
"""
from __future__ import annotations

import torch


def add_rmsnorm(x: torch.Tensor, weight: torch.Tensor, y: torch.Tensor | None = None, eps: float = 1e-6):
    """Returns (x_new, normed); every intermediate is rounded to ``x.dtype`` where the eager reference rounds."""
    dt = x.dtype
    if y is not None:
        x = (x.float() + y.float()).to(dt)
    xf = x.float()
    n = (xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)).to(dt)
    return x, (n.float() * weight.float()).to(dt)


def headnorm_gate(h: torch.Tensor, o_preact: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6):
    """h (B,NH,S,DH), o_preact (B,S,NH*DH), weight (NH*DH,) -> (B,S,NH*DH)."""
    dt = h.dtype
    B, NH, S, DH = h.shape
    hf = h.transpose(1, 2).float()                                   # (B,S,NH,DH)
    c = hf - hf.mean(dim=-1, keepdim=True)
    n = (c * torch.rsqrt(hf.var(dim=-1, keepdim=True, unbiased=False) + eps)).to(dt)
    nw = (n.reshape(B, S, NH * DH).float() * weight.float()).to(dt)
    g = torch.sigmoid(o_preact.float()).to(dt)
    return (g.float() * nw.float()).to(dt)


def soft_cap(x: torch.Tensor, cap: float, out_float32: bool = False):
    dt = x.dtype
    q = (x.float() / cap).to(dt)
    t = torch.tanh(q.float()).to(dt)
    y = (cap * t.float()).to(dt)
    return y.float() if out_float32 else y
