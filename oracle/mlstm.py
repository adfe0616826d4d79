"""CPU oracle for the mLSTM recurrent cell -- TEST INFRASTRUCTURE, NOT PRODUCT.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import this module; the product package never does.

This is a restatement, in plain PyTorch on the CPU, of the mLSTM cell
arithmetic that the reference selects with the kernel names
``chunkwise--native_autograd`` / ``native_sequence__native`` / ``native``.
Those kernels live in the third-party package ``mlstm_kernels`` (declared,
unpinned, in the reference's ``pyproject.toml:40`` / ``setup.cfg:41`` and
imported at ``xlstm/xlstm_large/model.py:3-14``), which is not vendored in
the reference tree.  The same arithmetic exists inside the reference at

* ``xlstm/blocks/mlstm/backends.py:93-146``  (stabilised recurrent step),
* ``xlstm/blocks/mlstm/backends.py:149-263`` (chunkwise form),
* ``xlstm/blocks/mlstm/backends.py:9-90``    (quadratic parallel form),

and this file follows those equations with two deliberate generalisations:
(i) the query/key width DHQK may differ from the value width DHV, and
(ii) the ``1/sqrt(DHQK)`` factor sits on the *query* in every function, so
that C and n hold un-scaled keys (``backends.py:168`` does this in the
chunkwise form; the step function at ``backends.py:134-137`` scales k instead,
which changes C and n by sqrt(DHQK) but not h).

Pinning: the reference's own tests at this boundary are self-consistency
checks only (no golden vectors).  ``tests/golden/make_golden.py`` runs the
reference's ``chunkwise_simple`` / ``recurrent_step_stabilized_simple`` /
``parallel_stabilized_simple`` in this container and commits their outputs;
``tests/test_oracle_mlstm.py`` checks this restatement against them.

State convention: C (B,NH,DHQK,DHV), n (B,NH,DHQK), m (B,NH,1), all fp32;
an absent / reset state is C=0, n=0, m=0 (``backends.py:185-194``).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def _state_or_zeros(c, n, m, B, NH, DHQK, DHV, device):
    f32 = torch.float32
    c = torch.zeros(B, NH, DHQK, DHV, dtype=f32, device=device) if c is None else c.to(f32)
    n = torch.zeros(B, NH, DHQK, dtype=f32, device=device) if n is None else n.to(f32)
    m = torch.zeros(B, NH, 1, dtype=f32, device=device) if m is None else m.to(f32).reshape(B, NH, 1)
    return c, n, m


def mlstm_step(q, k, v, i, f, c=None, n=None, m=None, eps: float = 1e-6):
    """One token of the stabilised recurrence (``backends.py:126-144``).

    q,k (B,NH,DHQK); v (B,NH,DHV); i,f (B,NH,1) or (B,NH).
    Returns h (B,NH,DHV) in fp32 and the new (c,n,m).
    """
    B, NH, DHQK = q.shape
    DHV = v.shape[-1]
    c, n, m = _state_or_zeros(c, n, m, B, NH, DHQK, DHV, q.device)
    q32, k32, v32 = q.float(), k.float(), v.float()
    i32 = i.float().reshape(B, NH, 1)
    logf = F.logsigmoid(f.float().reshape(B, NH, 1))

    m_new = torch.maximum(logf + m, i32)
    f_act = torch.exp(logf + m - m_new)
    i_act = torch.exp(i32 - m_new)

    c_new = f_act[..., None] * c + i_act[..., None] * (k32[..., :, None] * v32[..., None, :])
    n_new = f_act * n + i_act * k32

    qs = q32 * (DHQK ** -0.5)
    num = torch.einsum("bhd,bhde->bhe", qs, c_new)
    qn = (qs * n_new).sum(-1, keepdim=True)
    den = torch.maximum(qn.abs(), torch.exp(-m_new)) + eps
    return num / den, (c_new, n_new, m_new)


def mlstm_sequence(q, k, v, i, f, c=None, n=None, m=None, eps: float = 1e-6):
    """Token-by-token recurrence over S tokens: the sequence kernel's contract.

    q,k (B,NH,S,DHQK); v (B,NH,S,DHV); i,f (B,NH,S).  Returns h (B,NH,S,DHV)
    fp32 and the last (c,n,m).
    """
    B, NH, S, DHQK = q.shape
    DHV = v.shape[-1]
    state = _state_or_zeros(c, n, m, B, NH, DHQK, DHV, q.device)
    hs = []
    for t in range(S):
        h, state = mlstm_step(q[:, :, t], k[:, :, t], v[:, :, t], i[:, :, t], f[:, :, t], *state, eps=eps)
        hs.append(h)
    if hs:
        h = torch.stack(hs, dim=2)
    else:
        h = torch.zeros(B, NH, 0, DHV)
    return h, state


def mlstm_chunkwise(q, k, v, i, f, c=None, n=None, m=None, chunk_size: int = 64, eps: float = 1e-6):
    """Chunkwise-parallel form (``backends.py:173-258``), S % chunk_size == 0.

    All arithmetic in fp32 whatever the input dtype; returns fp32 h and the
    last (c,n,m).  Written as an explicit scan over chunks so that only one
    C state is alive at a time (the reference materialises all NC+1 of them).
    """
    B, NH, S, DHQK = q.shape
    DHV = v.shape[-1]
    L = chunk_size
    assert S % L == 0, "chunkwise form needs S to be a multiple of the chunk size"
    NC = S // L
    c, n, m = _state_or_zeros(c, n, m, B, NH, DHQK, DHV, q.device)
    m = m.reshape(B, NH)

    qs = q.float().reshape(B, NH, NC, L, DHQK) * (DHQK ** -0.5)
    kc = k.float().reshape(B, NH, NC, L, DHQK)
    vc = v.float().reshape(B, NH, NC, L, DHV)
    ic = i.float().reshape(B, NH, NC, L)
    logf = F.logsigmoid(f.float()).reshape(B, NH, NC, L)
    b = logf.cumsum(-1)                      # b_j   (backends.py:176)
    g = b[..., -1]                           # chunk total forget
    causal = torch.tril(torch.ones(L, L, dtype=torch.bool, device=q.device))

    out = torch.empty(B, NH, NC, L, DHV, dtype=torch.float32, device=q.device)
    for kappa in range(NC):
        bk, ik, gk = b[:, :, kappa], ic[:, :, kappa], g[:, :, kappa]
        # ---- intra-chunk decay matrix and per-row stabiliser (backends.py:220-233)
        logD = bk[..., :, None] - bk[..., None, :] + ik[..., None, :]
        logD = logD.masked_fill(~causal, float("-inf"))
        m_row = torch.maximum(logD.max(-1).values, bk + m[..., None])          # (B,NH,L)
        inter_scale = torch.exp(bk + m[..., None] - m_row)                       # (B,NH,L)
        Dm = torch.exp(logD - m_row[..., None])
        S_qk = qs[:, :, kappa] @ kc[:, :, kappa].transpose(-1, -2)
        E = S_qk * Dm
        num = E @ vc[:, :, kappa] + inter_scale[..., None] * (qs[:, :, kappa] @ c)
        qn = E.sum(-1) + inter_scale * torch.einsum("bhld,bhd->bhl", qs[:, :, kappa], n)
        den = torch.maximum(qn.abs(), torch.exp(-m_row)) + eps
        out[:, :, kappa] = num / den[..., None]
        # ---- carry the state across the chunk (backends.py:177-218)
        a = gk[..., None] - bk + ik                                              # (B,NH,L)
        m_next = torch.maximum(gk + m, a.max(-1).values)
        decay = torch.exp(gk + m - m_next)
        w = torch.exp(a - m_next[..., None])                                     # (B,NH,L)
        kw = kc[:, :, kappa] * w[..., None]
        c = decay[..., None, None] * c + kw.transpose(-1, -2) @ vc[:, :, kappa]
        n = decay[..., None] * n + kw.sum(-2)
        m = m_next
    return out.reshape(B, NH, S, DHV), (c, n, m.reshape(B, NH, 1))


def mlstm_parallel(q, k, v, i, f, eps: float = 1e-6):
    """Quadratic form from a zero state (``backends.py:9-90``); h only."""
    B, NH, S, DHQK = q.shape
    logf = F.logsigmoid(f.float())
    b = logf.cumsum(-1)
    logD = b[..., :, None] - b[..., None, :] + i.float()[..., None, :]
    causal = torch.tril(torch.ones(S, S, dtype=torch.bool, device=q.device))
    logD = logD.masked_fill(~causal, float("-inf"))
    # with a zero initial state the stabiliser also covers m_0 = 0 decayed by b_j
    m_row = torch.maximum(logD.max(-1).values, b)
    Dm = torch.exp(logD - m_row[..., None])
    E = (q.float() * DHQK ** -0.5) @ k.float().transpose(-1, -2) * Dm
    den = torch.maximum(E.sum(-1).abs(), torch.exp(-m_row)) + eps
    return (E @ v.float()) / den[..., None]


def mlstm_inference(q, k, v, i, f, c=None, n=None, m=None, chunk_size: int = 64, eps: float = 1e-6):
    """The backend's ``inference`` mode: chunkwise on the largest multiple of the
    chunk size, the recurrence on the remaining < chunk_size tokens, the step
    function when S == 1 (contract documented at ``model.py:56-75``)."""
    B, NH, S, DHQK = q.shape
    if S == 0:
        return torch.zeros(B, NH, 0, v.shape[-1]), _state_or_zeros(c, n, m, B, NH, DHQK, v.shape[-1], q.device)
    if S == 1:
        h, st = mlstm_step(q[:, :, 0], k[:, :, 0], v[:, :, 0], i[:, :, 0], f[:, :, 0], c, n, m, eps=eps)
        return h[:, :, None], st
    S0 = (S // chunk_size) * chunk_size
    parts = []
    state = (c, n, m)
    if S0 > 0:
        h0, state = mlstm_chunkwise(q[:, :, :S0], k[:, :, :S0], v[:, :, :S0], i[:, :, :S0], f[:, :, :S0],
                                    *state, chunk_size=chunk_size, eps=eps)
        parts.append(h0)
    if S0 < S:
        h1, state = mlstm_sequence(q[:, :, S0:], k[:, :, S0:], v[:, :, S0:], i[:, :, S0:], f[:, :, S0:],
                                   *state, eps=eps)
        parts.append(h1)
    return torch.cat(parts, dim=2), state


def mlstm_packed(q, k, v, i, f, cu_seqlens, chunk_size: int = 64, eps: float = 1e-6):
    """Packed ragged batch: every document starts from the zero state.

    q,k (NH,T,DHQK), v (NH,T,DHV), i,f (NH,T) over the flattened token axis
    T = cu_seqlens[-1]; document d owns tokens [cu_seqlens[d], cu_seqlens[d+1]).
    The reference has no packed path, so the oracle is by definition "run each
    document alone through the native inference path and concatenate".
    Returns h (NH,T,DHV) and per-document final states stacked on dim 0:
    c (ND,NH,DHQK,DHV), n (ND,NH,DHQK), m (ND,NH,1).
    """
    cu = [int(x) for x in cu_seqlens]
    hs, cs, ns, ms = [], [], [], []
    for d in range(len(cu) - 1):
        s, e = cu[d], cu[d + 1]
        h, (c, n, m) = mlstm_inference(q[None, :, s:e], k[None, :, s:e], v[None, :, s:e],
                                       i[None, :, s:e], f[None, :, s:e], chunk_size=chunk_size, eps=eps)
        hs.append(h[0]); cs.append(c[0]); ns.append(n[0]); ms.append(m[0])
    return torch.cat(hs, dim=1), (torch.stack(cs), torch.stack(ns), torch.stack(ms))
