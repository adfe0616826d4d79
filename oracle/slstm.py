"""CPU oracle for the sLSTM recurrent cell -- TEST INFRASTRUCTURE, NOT PRODUCT.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import this module; the product package never does.

Restates, in plain PyTorch on the CPU, the reference's sLSTM recurrence:

* time loop and recurrent product ``xlstm/blocks/slstm/src/vanilla/__init__.py:17-74``
  (``Ry[b, g, head, d_out] = sum_{d_in} h[b, head, d_in] * R[head, d_in, g, d_out]``),
* pointwise update ``xlstm/blocks/slstm/src/vanilla/slstm.py:8-37`` and its CUDA
  twin ``xlstm/blocks/slstm/src/cuda/slstm_pointwise.cu:24-116``.

The two reference backends differ in one rule: the vanilla code takes the
"fresh state" branch ``m' = i`` only when the WHOLE n tensor is zero
(``slstm.py:25``) while the CUDA kernel tests each element
(``slstm_pointwise.cu:79``).  ``fresh_rule`` selects which one is restated;
they coincide whenever all rows start fresh or none do.  With document
resets inside a packed row only the per-element rule is meaningful.

Layouts (the cell's external ones, ``xlstm/blocks/slstm/cell.py:234-261, 339-342``):
input ``wx`` (B,S,4*H) gate-major: [i | f | z | o], each block (NH,DH) ordered;
R (NH, DH_in, 4, DH_out); bias (NH, 4, DH); state (4,B,H) ordered (h,c,n,m).

Pinning: ``tests/golden/make_golden.py`` runs the reference's vanilla cell in
this container and commits its outputs; ``tests/test_oracle_slstm.py`` checks
this restatement against them.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def slstm_pointwise(raw, state, fresh_rule: str = "elementwise", stabiliser_grad: bool = True):
    """raw (B,4,H) pre-activations (i,f,z,o); state (4,B,H) = (h,c,n,m). fp32.  The function is differentiable (plain
    torch operators), which makes autograd over it the oracle of the backward pass; with ``stabiliser_grad=False``
    the new m is a constant of the step, the rule of the reference's backward kernel
    (``slstm_pointwise.cu:118-196`` never differentiates m and returns a zero gradient for it) -- the two agree for
    any loss on h, which does not depend on the stabiliser."""
    _, c, n, m = state.unbind(0)
    i_raw, f_raw, z_raw, o_raw = raw.unbind(1)
    logf_plus_m = m + F.logsigmoid(f_raw)
    if fresh_rule == "elementwise":
        m_new = torch.where(n == 0.0, i_raw, torch.maximum(i_raw, logf_plus_m))
    elif fresh_rule == "whole_tensor":
        m_new = i_raw if bool(torch.all(n == 0.0)) else torch.maximum(i_raw, logf_plus_m)
    else:
        raise ValueError(fresh_rule)
    if not stabiliser_grad:
        m_new = m_new.detach()
    i_gate = torch.exp(i_raw - m_new).clamp(max=1.0)
    f_gate = torch.exp(logf_plus_m - m_new).clamp(max=1.0)
    c_new = f_gate * c + i_gate * torch.tanh(z_raw)
    n_new = f_gate * n + i_gate
    h_new = torch.sigmoid(o_raw) * c_new / n_new
    return torch.stack((h_new, c_new, n_new, m_new), 0)


def slstm_forward(wx, R, bias, state=None, reset=None, fresh_rule: str = "elementwise",
                  state_dtype: torch.dtype = torch.float32, stabiliser_grad: bool = True):
    """Full sequence.

    wx (B,S,4H); R (NH,DH,4,DH); bias (NH,4,DH); state (4,B,H) or None;
    reset: optional bool (B,S), True where a new document starts (state is
    zeroed before that step).  ``state_dtype`` is the dtype the four states are
    rounded to after every step (the reference keeps them in the input dtype,
    ``vanilla/__init__.py:67-69`` and ``slstm_pointwise.cu:112-115``; fp32 means
    no rounding).  Returns h sequence (B,NH,S,DH) fp32 and final state (4,B,H).
    """
    B, S, H4 = wx.shape
    NH, DH = R.shape[0], R.shape[1]
    H = NH * DH
    assert H4 == 4 * H
    R32 = R.float().reshape(NH, DH, 4 * DH)
    b32 = bias.float().reshape(NH, 4, DH).permute(1, 0, 2).reshape(1, 4, H)
    st = torch.zeros(4, B, H) if state is None else state.float().clone()
    wx32 = wx.float().reshape(B, S, 4, H)
    hs = []
    for t in range(S):
        if reset is not None:
            st = torch.where(reset[:, t].reshape(1, B, 1), torch.zeros_like(st), st)
        h = st[0].reshape(B, NH, 1, DH)
        ry = (h @ R32[None]).reshape(B, NH, 4, DH).permute(0, 2, 1, 3).reshape(B, 4, H)
        st = slstm_pointwise(wx32[:, t] + ry + b32, st, fresh_rule, stabiliser_grad).to(state_dtype).float()
        hs.append(st[0])
    out = torch.stack(hs, 0).reshape(S, B, NH, DH).permute(1, 2, 0, 3).contiguous()
    return out, st
