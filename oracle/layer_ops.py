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

* ``causal_conv1d``: the depthwise causal convolution in front of the sLSTM cell (``CausalConv1d.forward``,
  ``xlstm/components/conv.py:110-129``: ``nn.Conv1d`` with ``groups = features`` and left padding ``K - 1``) followed by
  the layer's SiLU (``xlstm/blocks/slstm/layer.py:133-142``); with document offsets every document is convolved alone,
  which is what the reference gives when it is called once per document.

Pinning: ``tests/golden/make_golden_conv.py`` ran the reference's ``CausalConv1d`` (per document for the packed case);
``tests/golden/make_golden_layer.py`` ran the reference's own ``RMSNorm`` and ``MultiHeadLayerNorm``
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


def swiglu(gz: torch.Tensor):
    """silu(gz[..., :F]) * gz[..., F:] with the eager sequence's rounding (``act_fn(proj_up_gate(x)) * proj_up(x)``,
    xlstm/xlstm_large/model.py:268-277)."""
    dt = gz.dtype
    g, z = gz.chunk(2, dim=-1)
    return (torch.nn.functional.silu(g.float()).to(dt).float() * z.float()).to(dt)


def soft_cap(x: torch.Tensor, cap: float, out_float32: bool = False, bias: torch.Tensor | None = None):
    dt = x.dtype
    if bias is not None:   # a Linear layer's bias, rounded with its output
        x = (x.float() + bias.float()).to(dt)
    q = (x.float() / cap).to(dt)
    t = torch.tanh(q.float()).to(dt)
    y = (cap * t.float()).to(dt)
    return y.float() if out_float32 else y


def causal_conv1d(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None, cu_seqlens=None, silu: bool = True):
    """x (B,S,F), weight (F,K) [= nn.Conv1d(groups=F).weight[:,0,:]], bias (F).  out[b,t] = bias + sum_j weight[:,j] *
    x[b, t-(K-1)+j] with zeros in front of the first token of the document (of the row without ``cu_seqlens``), rounded
    to ``x.dtype``; then SiLU, rounded again."""
    dt = x.dtype
    B, S, F_ = x.shape
    K = weight.shape[1]
    xf = x.float().reshape(B * S, F_)
    cu = [b * S for b in range(B + 1)] if cu_seqlens is None else sorted(set([int(c) for c in cu_seqlens] + [b * S for b in range(B + 1)]))
    out = torch.zeros_like(xf)
    for a, e in zip(cu[:-1], cu[1:]):
        if e <= a:
            continue
        seg = xf[a:e]
        acc = torch.zeros_like(seg) if bias is None else bias.float().expand_as(seg).clone()
        for lag in range(K):
            if lag < e - a:
                acc[lag:] += seg[:e - a - lag] * weight[:, K - 1 - lag].float()
        out[a:e] = acc
    y = out.to(dt)
    if silu:
        y = torch.nn.functional.silu(y.float()).to(dt)
    return y.reshape(B, S, F_)


def head_group_norm(h: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5):
    """h (B,NH,S,DH), weight (NH*DH,) [already 1 + residual weight] -> (B,S,NH*DH): ``F.group_norm`` over every head of
    every token, rounded once (``MultiHeadLayerNorm.forward``, xlstm/components/ln.py:52-68)."""
    dt = h.dtype
    B, NH, S, DH = h.shape
    hf = h.transpose(1, 2).float()
    c = hf - hf.mean(dim=-1, keepdim=True)
    n = c * torch.rsqrt(hf.var(dim=-1, keepdim=True, unbiased=False) + eps)
    return (n.reshape(B, S, NH * DH) * weight.float()).to(dt)


def headwise_proj(inputs, weights, in_sel=None):
    """``LinearHeadwiseExpand.forward`` per slot (xlstm/components/linear_headwise.py:75-82, no bias) and the concatenation
    of the sLSTM layer (xlstm/blocks/slstm/layer.py:145-154): inputs (..., NH*DH), weights (NH, DH_out, DH_in) each;
    fp32 accumulation, one rounding to the input dtype; result (..., n * NH * DH_out), slot-major."""
    if isinstance(inputs, torch.Tensor):
        inputs = [inputs]
    in_sel = [0] * len(weights) if in_sel is None else list(in_sel)
    outs = []
    for w, sel in zip(weights, in_sel):
        x = inputs[sel]
        NH = w.shape[0]
        xh = x.float().reshape(*x.shape[:-1], NH, -1)
        y = torch.einsum("...hd,hod->...ho", xh, w.float())
        outs.append(y.reshape(*x.shape[:-1], -1).to(x.dtype))
    return torch.cat(outs, dim=-1)
