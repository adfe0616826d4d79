"""Tensor-level entry points: unpack torch tensors, call the C ABI on the current CUDA stream.

PyTorch is used for device memory and streams only; all arithmetic happens in
the sm_100a kernels behind ``include/xlstm_b200.h``.  Nothing here falls back
to PyTorch math: unsupported inputs raise.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from . import _lib
from ._lib import (AddRmsnormParams, Conv1dParams, HeadwiseParams, GreedyParams, HeadnormGateParams, MlstmDecodeCellParams, MlstmSeqParams, MlstmStepParams, SlstmParams, SlstmBwdParams, SoftCapParams, SwigluParams, XL_BF16, XL_F32,
                   check, lib)

_DTYPES = {torch.float32: XL_F32, torch.bfloat16: XL_BF16}
_status_words: dict[int, torch.Tensor] = {}


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def status_word(device) -> torch.Tensor:
    """Per-device int32 word that kernels set when one of their bounded waits expires."""
    idx = torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    if idx not in _status_words:
        _status_words[idx] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{idx}")
    return _status_words[idx]


def check_device_status(device=None) -> None:
    """Synchronising check of the status word; raises if a kernel gave up on a wait."""
    w = status_word(device if device is not None else torch.cuda.current_device())
    v = int(w.item())
    if v != 0:
        w.zero_()
        raise RuntimeError(f"xlstm_b200 kernel reported device status {v} (a bounded wait expired)")


def _require_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise ValueError("xlstm_b200 kernels need CUDA tensors (there is no CPU path)")


def _last_contig(t: torch.Tensor) -> torch.Tensor:
    return t if t.stride(-1) == 1 else t.contiguous()


def _gate(t: torch.Tensor) -> torch.Tensor:
    return t if t.dtype == torch.float32 else t.float()


def prepare_cu_seqlens(cu_seqlens, B: int, S: int, device) -> tuple[torch.Tensor, int]:
    """Validate document offsets on the host and return (int32 device tensor, num_docs).

    Offsets index the flattened (B*S) token axis; they must start at 0, end at B*S, be
    non-decreasing, and no document may straddle two rows.  A tensor that already lives on
    the device is trusted as is (validating it would force a synchronisation).
    """
    if torch.is_tensor(cu_seqlens) and cu_seqlens.is_cuda:
        if cu_seqlens.dtype != torch.int32:
            raise ValueError("cu_seqlens on the device must be int32")
        return cu_seqlens.contiguous(), cu_seqlens.numel() - 1
    cu = [int(x) for x in (cu_seqlens.tolist() if torch.is_tensor(cu_seqlens) else cu_seqlens)]
    if len(cu) < 2 or cu[0] != 0 or cu[-1] != B * S:
        raise ValueError(f"cu_seqlens must start at 0 and end at B*S={B * S}, got {cu[:1]}..{cu[-1:]}")
    for a, b in zip(cu[:-1], cu[1:]):
        if b < a:
            raise ValueError("cu_seqlens must be non-decreasing")
        if b > a and (a // S) != ((b - 1) // S):
            raise ValueError(f"document [{a},{b}) straddles two rows of length {S}")
    return torch.tensor(cu, dtype=torch.int32, device=device), len(cu) - 1


def mlstm_sequence(q, k, v, i, f, c_initial=None, n_initial=None, m_initial=None, cu_seqlens=None,
                   eps: float = 1e-6, kernel: str = "auto"):
    """mLSTM over a sequence.  q,k (B,NH,S,DHQK), v (B,NH,S,DHV), i,f (B,NH,S).

    kernel: "chunkwise" (tcgen05), "recurrent" (fp32 recurrence) or "auto" (chunkwise when the
    shape/dtype is covered by it, else recurrent).  Returns h (B,NH,S,DHV) in q's dtype and the final
    fp32 state (c,n,m) with one row per document: c (N,NH,DHQK,DHV), n (N,NH,DHQK), m (N,NH,1).
    """
    _require_cuda(q, k, v, i, f, c_initial, n_initial, m_initial)
    if q.dtype not in _DTYPES or k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError(f"q,k,v must share a dtype in {list(_DTYPES)}, got {q.dtype},{k.dtype},{v.dtype}")
    B, NH, S, DHQK = q.shape
    DHV = v.shape[-1]
    if k.shape != q.shape or v.shape[:3] != q.shape[:3] or i.shape != (B, NH, S) or f.shape != (B, NH, S):
        raise ValueError("inconsistent shapes for q,k,v,i,f")
    dev = q.device
    q, k, v = _last_contig(q), _last_contig(k), _last_contig(v)
    i, f = _gate(i), _gate(f)
    if i.stride() != f.stride():
        i, f = i.contiguous(), f.contiguous()
    chunk_ok = (q.dtype == torch.bfloat16 and DHQK in (64, 128, 256) and DHV % 128 == 0
                and all(s % 8 == 0 for t in (q, k, v) for s in t.stride()[:3])
                and all(t.data_ptr() % 16 == 0 for t in (q, k, v)))
    if kernel == "auto":
        kernel = "chunkwise" if chunk_ok else "recurrent"
    if kernel not in ("chunkwise", "recurrent"):
        raise ValueError(f"unknown kernel {kernel!r}")

    cu_dev, nd = (None, B)
    if cu_seqlens is not None:
        cu_dev, nd = prepare_cu_seqlens(cu_seqlens, B, S, dev)
    have0 = c_initial is not None
    if have0:
        if n_initial is None or m_initial is None:
            raise ValueError("c_initial, n_initial and m_initial must be given together")
        c0 = c_initial.float().contiguous()
        n0 = n_initial.float().contiguous()
        m0 = m_initial.float().contiguous()
        if c0.shape != (nd, NH, DHQK, DHV) or n0.shape != (nd, NH, DHQK) or m0.numel() != nd * NH:
            raise ValueError("initial state shapes must be (N,NH,DHQK,DHV), (N,NH,DHQK), (N,NH[,1])")
    h = torch.empty(B, NH, S, DHV, dtype=q.dtype, device=dev)
    c = torch.empty(nd, NH, DHQK, DHV, dtype=torch.float32, device=dev)
    n = torch.empty(nd, NH, DHQK, dtype=torch.float32, device=dev)
    m = torch.empty(nd, NH, 1, dtype=torch.float32, device=dev)

    p = MlstmSeqParams()
    p.q, p.k, p.v, p.h = q.data_ptr(), k.data_ptr(), v.data_ptr(), h.data_ptr()
    p.igate, p.fgate = i.data_ptr(), f.data_ptr()
    if have0:
        p.c0, p.n0, p.m0 = c0.data_ptr(), n0.data_ptr(), m0.data_ptr()
    p.c_out, p.n_out, p.m_out = c.data_ptr(), n.data_ptr(), m.data_ptr()
    p.cu_seqlens = cu_dev.data_ptr() if cu_dev is not None else None
    p.status = status_word(dev).data_ptr()
    p.B, p.NH, p.S, p.DHQK, p.DHV, p.num_docs = B, NH, S, DHQK, DHV, nd
    p.q_sb, p.q_sh, p.q_st = q.stride()[:3]
    p.k_sb, p.k_sh, p.k_st = k.stride()[:3]
    p.v_sb, p.v_sh, p.v_st = v.stride()[:3]
    p.h_sb, p.h_sh, p.h_st = h.stride()[:3]
    p.g_sb, p.g_sh, p.g_st = i.stride()
    p.eps, p.dtype = eps, _DTYPES[q.dtype]
    fn = lib().xl_mlstm_chunkwise if kernel == "chunkwise" else lib().xl_mlstm_recurrent
    with torch.cuda.device(dev):
        check(fn(C.byref(p), _stream_ptr(dev)), f"xl_mlstm_{kernel}")
    return h, (c, n, m)


_host_streams: dict[int, list] = {}


def mlstm_sequence_from_host(q, k, v, i, f, h_out, c_out, n_out=None, m_out=None, device=None, head_groups: Optional[int] = None,
                             eps: float = 1e-6):
    """Prefill whose inputs and outputs live in pinned HOST memory: q, k ``(B,NH,S,DHQK)``, v ``(B,NH,S,DHV)``, gates
    ``(B,NH,S)`` in, ``h_out (B,NH,S,DHV)``, ``c_out (B,NH,DHQK,DHV)`` (optionally n, m) out, zero initial state.

    Heads and batch rows are independent, so the call is cut into ``B x head_groups`` contiguous pieces that go round
    three streams: the upload of one piece overlaps the kernel and the download of the pieces before it (the link is
    full duplex), and the whole call takes about as long as its uploads alone.  Returns when everything is enqueued;
    the caller's current stream waits for the last piece."""
    dev = torch.device(device if device is not None else "cuda")
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    dev = torch.device("cuda", idx)
    B, NH = q.shape[0], q.shape[1]
    if head_groups is None:   # pieces of a few tens of MB keep the link busy in both directions (measured: 4 groups of 2 heads at
        head_groups = next(g for g in (4, 2, 1) if NH % g == 0)   # the 7B head shape: 11.9 ms per 32 768 tokens; 2: 12.1; 8: 14.2)
    if NH % head_groups:
        raise ValueError(f"num_heads={NH} is not divisible by head_groups={head_groups}")
    for t in (q, k, v, i, f, h_out, c_out):
        if t.device.type != "cpu" or not t.is_pinned():
            raise ValueError("mlstm_sequence_from_host wants pinned host tensors")
    streams = _host_streams.setdefault(idx, [torch.cuda.Stream(device=dev) for _ in range(3)])
    cur = torch.cuda.current_stream(dev)
    for st in streams:
        st.wait_stream(cur)
    hg = NH // head_groups
    piece = 0
    for b in range(B):
        for g in range(head_groups):
            sl = (slice(b, b + 1), slice(g * hg, (g + 1) * hg))
            st = streams[piece % len(streams)]
            piece += 1
            with torch.cuda.stream(st):
                dq, dk, dv, di, df = [t[sl].to(dev, non_blocking=True) for t in (q, k, v, i, f)]
                h, (c, n, m) = mlstm_sequence(dq, dk, dv, di, df, kernel="chunkwise", eps=eps)
                h_out[sl].copy_(h, non_blocking=True)
                c_out[sl].copy_(c, non_blocking=True)
                if n_out is not None:
                    n_out[sl].copy_(n, non_blocking=True)
                if m_out is not None:
                    m_out[sl].copy_(m, non_blocking=True)
                for t in (dq, dk, dv, di, df, h, c, n, m):
                    t.record_stream(st)
    for st in streams:
        cur.wait_stream(st)


def prepare_slots(slot, B: int, n_slots: int, device) -> torch.Tensor:
    """Pool rows of the B decode streams as the int32 device vector the step kernel reads.

    A host tensor or list is checked here: one entry per stream, every entry below ``n_slots``, no row named by two
    active streams (negative entries mark inactive streams and may repeat).  A tensor that already lives on the device
    must be a (B,) integer vector; its values cannot be inspected without a synchronisation, so the kernel itself
    skips entries outside the pool and reports them through the status word (``check_device_status``)."""
    if torch.is_tensor(slot) and slot.is_cuda:
        if slot.dim() != 1 or slot.numel() != B or slot.dtype not in (torch.int32, torch.int64):
            raise ValueError(f"slot must be a ({B},) int32 (or int64) vector, got {tuple(slot.shape)} {slot.dtype}")
        if slot.device != torch.device(device):
            raise ValueError("slot lives on another device than the inputs")
        return slot.to(torch.int32).contiguous()
    vals = [int(x) for x in (slot.tolist() if torch.is_tensor(slot) else slot)]
    if len(vals) != B:
        raise ValueError(f"slot must have one entry per stream ({B}), got {len(vals)}")
    active = [x for x in vals if x >= 0]
    if any(x >= n_slots for x in active):
        raise ValueError(f"slot entries must be below the pool size {n_slots}")
    if len(set(active)) != len(active):
        raise ValueError("two active streams name the same pool row")
    return torch.tensor(vals, dtype=torch.int32, device=device)


def _step_state_params(p, q, k, v, c, n, m, slot, eps, inplace):
    """Fills the part of ``MlstmStepParams`` that the plain step and the fused decode cell share (inputs, state pool,
    slots); returns the output state tensors and the (possibly converted) tensors that must stay alive for the launch."""
    B, NH, DHQK = q.shape
    DHV = v.shape[-1]
    dev = q.device
    if slot is not None:
        if c is None:
            raise ValueError("`slot` addresses rows of a state pool: pass c, n, m")
        slot = prepare_slots(slot, B, c.shape[0], dev)
    q, k, v = _last_contig(q), _last_contig(k), _last_contig(v)
    have = c is not None
    if have:
        if c.dtype != torch.float32 or not c.is_contiguous() or not n.is_contiguous():
            raise ValueError("state pool must be contiguous fp32")
        N = c.shape[0]
        m = m.reshape(N, NH, 1)
        if not m.is_contiguous():
            m = m.contiguous()
        if slot is None and N != B:
            raise ValueError("without `slot` the state pool must have one row per stream")
    else:
        N = B
    c_out = c if (have and inplace) else torch.empty(N, NH, DHQK, DHV, dtype=torch.float32, device=dev)
    if have and not inplace and slot is not None:
        c_out.copy_(c)  # rows not addressed by `slot` keep their contents
    n_out = n.clone() if (have and slot is not None) else torch.empty(N, NH, DHQK, dtype=torch.float32, device=dev)
    m_out = m.clone() if (have and slot is not None) else torch.empty(N, NH, 1, dtype=torch.float32, device=dev)
    p.q, p.k, p.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    if have:
        p.c_in, p.n_in, p.m_in = c.data_ptr(), n.data_ptr(), m.data_ptr()
    p.c_out, p.n_out, p.m_out = c_out.data_ptr(), n_out.data_ptr(), m_out.data_ptr()
    p.slot = slot.data_ptr() if slot is not None else None
    p.status = status_word(dev).data_ptr()
    p.B, p.NH, p.DHQK, p.DHV, p.n_slots = B, NH, DHQK, DHV, N
    p.q_sb, p.q_sh = q.stride()[:2]
    p.k_sb, p.k_sh = k.stride()[:2]
    p.v_sb, p.v_sh = v.stride()[:2]
    p.eps, p.dtype = eps, _DTYPES[q.dtype]
    return (c_out, n_out, m_out), (q, k, v, m, slot)


def mlstm_step(q, k, v, i, f, c, n, m, slot=None, eps: float = 1e-6, inplace: bool = True):
    """One decode step.  q,k (B,NH,DHQK), v (B,NH,DHV), i,f (B,NH[,1]); state pool c (N,NH,DHQK,DHV),
    n (N,NH,DHQK), m (N,NH[,1]) fp32; ``slot`` (B,) selects each stream's pool row (default: row b; a negative
    entry marks an inactive stream whose pool rows stay untouched; see :func:`prepare_slots`).

    With ``inplace`` the large C state is updated where it lives and the SAME tensor object is returned,
    so a caller that copies the returned state back into its own buffers (xlstm_large/model.py:221-225)
    performs a no-op for C.  n and m are always returned as new small tensors (several thread blocks
    read the old values while one writes).  Without a pool (c is None) the state starts from zero.
    """
    _require_cuda(q, k, v, i, f, c, n, m)
    B, NH, _ = q.shape
    dev = q.device
    i, f = _gate(i).reshape(B, NH), _gate(f).reshape(B, NH)
    if i.stride() != f.stride():
        i, f = i.contiguous(), f.contiguous()
    p = MlstmStepParams()
    state, keep = _step_state_params(p, q, k, v, c, n, m, slot, eps, inplace)
    h = torch.empty(B, NH, v.shape[-1], dtype=q.dtype, device=dev)
    p.h = h.data_ptr()
    p.igate, p.fgate = i.data_ptr(), f.data_ptr()
    p.h_sb, p.h_sh = h.stride()[:2]
    p.g_sb, p.g_sh = i.stride()
    with torch.cuda.device(dev):
        check(lib().xl_mlstm_step(C.byref(p), _stream_ptr(dev)), "xl_mlstm_step")
    return h, state


def mlstm_decode_cell(q, k, v, gates_raw, gate_bias, gate_cap: float, ogate, norm_weight, c, n, m, slot=None,
                      eps: float = 1e-6, norm_eps: float = 1e-6):
    """The cell part of one decode step of the mLSTM layer in ONE kernel: soft cap of the gate pre-activations
    (xlstm/xlstm_large/model.py:389-394, fp32 arithmetic), the step of :func:`mlstm_step` (C updated in place), and the
    per-head norm + weight + output gate behind it (model.py:435-449).

    q,k (B,NH,DHQK), v (B,NH,DHV) as for the step; ``gates_raw`` (B, 2*NH): the projection's input-gate columns of all
    heads, then its forget-gate columns (a column slice of the stacked projection output is fine); ``gate_bias`` (2*NH)
    or None; ``ogate`` (B, NH*DHV); ``norm_weight`` (NH*DHV).  Returns (B, NH*DHV), the input of out_proj, and the
    state like :func:`mlstm_step`."""
    _require_cuda(q, k, v, gates_raw, gate_bias, ogate, norm_weight, c, n, m)
    B, NH, _ = q.shape
    DHV = v.shape[-1]
    dev, dt = q.device, q.dtype
    if DHV > 1024:
        raise ValueError("mlstm_decode_cell: head value width above 1024")
    gates_raw, ogate = _last_contig(gates_raw).reshape(B, 2 * NH), _last_contig(ogate).reshape(B, NH * DHV)
    if gates_raw.dtype != dt or ogate.dtype != dt or norm_weight.dtype != dt or (gate_bias is not None and gate_bias.dtype != dt):
        raise ValueError("mlstm_decode_cell: gates, output gate, bias and norm weight in the dtype of q")
    norm_weight = norm_weight.contiguous()
    if norm_weight.numel() != NH * DHV or (gate_bias is not None and gate_bias.numel() != 2 * NH):
        raise ValueError("mlstm_decode_cell: norm weight (NH*DHV), gate bias (2*NH)")
    f = MlstmDecodeCellParams()
    state, keep = _step_state_params(f.step, q, k, v, c, n, m, slot, eps, True)
    hg = torch.empty(B, NH * DHV, dtype=dt, device=dev)
    gate_bias = gate_bias.contiguous() if gate_bias is not None else None
    f.gates_raw, f.ogate, f.norm_weight, f.hg = gates_raw.data_ptr(), ogate.data_ptr(), norm_weight.data_ptr(), hg.data_ptr()
    f.gate_bias = gate_bias.data_ptr() if gate_bias is not None else None
    f.gr_sb, f.o_sb, f.hg_sb = gates_raw.stride(0), ogate.stride(0), hg.stride(0)
    f.gate_cap, f.norm_eps = float(gate_cap), float(norm_eps)
    with torch.cuda.device(dev):
        check(lib().xl_mlstm_decode_cell(C.byref(f), _stream_ptr(dev)), "xl_mlstm_decode_cell")
    return hg, state


def slstm_forward(wx, R, bias, state0=None, cu_seqlens=None, train_cache: bool = False):
    """sLSTM over a sequence.  wx (B,S,4*H) gate-major [i|f|z|o] each (NH,DH); R (NH,DH,4,DH); bias (NH,4,DH);
    state0 (4,B,H) ordered (h,c,n,m) or None.  Returns h (B,NH,S,DH) in wx's dtype and the final fp32 state; with
    ``train_cache`` also the opaque cache ``slstm_backward`` needs (no document offsets then)."""
    _require_cuda(wx, R, bias, state0)
    if wx.dtype != torch.bfloat16:
        raise ValueError("the sLSTM kernel computes on bf16 inputs (fp32 state); cast wx and R to bfloat16")
    B, S, H4 = wx.shape
    NH, DH = R.shape[0], R.shape[1]
    H = NH * DH
    if H4 != 4 * H or R.shape != (NH, DH, 4, DH) or bias.numel() != NH * 4 * DH:
        raise ValueError("inconsistent sLSTM shapes")
    dev = wx.device
    wx = wx.contiguous()
    R = R.to(torch.bfloat16).contiguous()
    bias = bias.float().contiguous()
    out = torch.empty(B, NH, S, DH, dtype=wx.dtype, device=dev)
    st = torch.empty(4, B, H, dtype=torch.float32, device=dev)
    p = SlstmParams()
    p.wx, p.R, p.bias = wx.data_ptr(), R.data_ptr(), bias.data_ptr()
    if state0 is not None:
        s0 = state0.float().contiguous()
        if s0.shape != (4, B, H):
            raise ValueError("state0 must be (4,B,H)")
        p.state0 = s0.data_ptr()
    p.h_out, p.state_out = out.data_ptr(), st.data_ptr()
    nd = 0
    if cu_seqlens is not None:
        cu_dev, nd = prepare_cu_seqlens(cu_seqlens, B, S, dev)
        p.cu_seqlens = cu_dev.data_ptr()
    p.status = status_word(dev).data_ptr()
    p.B, p.S, p.NH, p.DH, p.num_docs, p.dtype = B, S, NH, DH, nd, XL_BF16
    cache = None
    if train_cache:
        nbytes = lib().xl_slstm_cache_bytes(B, S, NH, DH)
        if nbytes <= 0:
            raise ValueError("the sLSTM training path needs a head size of 64, 128 or 256")
        cache = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        p.train_cache = cache.data_ptr()
    with torch.cuda.device(dev):
        check(lib().xl_slstm_forward(C.byref(p), _stream_ptr(dev)), "xl_slstm_forward")
    if train_cache:
        return out, st, cache
    return out, st


def slstm_backward(cache, R, dh, dstate_out=None, state0=None):
    """Backward through time of ``slstm_forward(..., train_cache=True)``: ``cache`` from that call, R (NH,DH,4,DH),
    dh (B,NH,S,DH) the gradient of its h, dstate_out (4,B,H) the gradient of its final state (m's entry is ignored)
    or None, state0 its initial state or None.  Returns dwx (B,S,4*H) in bf16 and dstate0 (4,B,H) fp32 (zero for m).
    Replaces sLSTMFunc.backward (xlstm/blocks/slstm/src/cuda/slstm.cc:137-254) up to the two sums ``slstm_weight_grads``
    forms."""
    _require_cuda(cache, R, dh, dstate_out, state0)
    B, NH, S, DH = dh.shape
    H = NH * DH
    if R.shape != (NH, DH, 4, DH):
        raise ValueError("inconsistent sLSTM shapes")
    dev = dh.device
    if cache.numel() != lib().xl_slstm_cache_bytes(B, S, NH, DH) or cache.dtype != torch.uint8:
        raise ValueError("cache does not belong to a forward call of these sizes")
    R = R.to(torch.bfloat16).contiguous()
    dh = dh.to(torch.bfloat16).contiguous()
    dwx = torch.empty(B, S, 4 * H, dtype=torch.bfloat16, device=dev)
    ds0 = torch.empty(4, B, H, dtype=torch.float32, device=dev)
    p = SlstmBwdParams()
    p.cache, p.R, p.dh, p.dwx, p.dstate0 = cache.data_ptr(), R.data_ptr(), dh.data_ptr(), dwx.data_ptr(), ds0.data_ptr()
    keep = []
    for name, t in (("dstate_out", dstate_out), ("state0", state0)):
        if t is not None:
            t32 = t.float().contiguous()
            if t32.shape != (4, B, H):
                raise ValueError(f"{name} must be (4,B,H)")
            keep.append(t32)
            setattr(p, name, t32.data_ptr())
    p.status = status_word(dev).data_ptr()
    p.B, p.S, p.NH, p.DH, p.dtype = B, S, NH, DH, XL_BF16
    with torch.cuda.device(dev):
        check(lib().xl_slstm_backward(C.byref(p), _stream_ptr(dev)), "xl_slstm_backward")
    return dwx, ds0


def slstm_weight_grads(dwx, h, state0=None):
    """Gradients of the recurrent matrix and the bias from the backward kernel's output: with h_{t-1} the forward's h
    shifted by one step (h_{-1} from state0), dR[n,k,g,u] = sum_{b,t} h_{t-1}[b,n,k] dwx[b,t,g,n,u] and
    dbias[n,g,u] = sum_{b,t} dwx[b,t,g,n,u] (the reference forms the same products after its time loop,
    slstm_backward.cu).  Plain batched matrix products, fp32 results: (NH,DH,4,DH) and (NH,4,DH)."""
    B, NH, S, DH = h.shape
    dw = dwx.reshape(B, S, 4, NH, DH)

    def mm(a, b):   # fp32 result; half-precision operands stay as they are where the GEMM library accumulates in fp32
        if a.is_cuda and a.dtype in (torch.bfloat16, torch.float16):
            try:
                return torch.bmm(a, b, out_dtype=torch.float32)
            except (TypeError, NotImplementedError, RuntimeError):
                pass
        return torch.bmm(a.float(), b.float())

    dR = torch.zeros(NH, DH, 4 * DH, dtype=torch.float32, device=dwx.device)
    if S > 1:   # steps 1 .. S-1 pair h_{t-1} = h[t-1] with dwx[t]: two shifted views, no shifted copy of h
        a = h[:, :, :-1].permute(1, 3, 0, 2).reshape(NH, DH, B * (S - 1)).to(dwx.dtype)      # (NH, DH_in, B*(S-1))
        b = dw[:, 1:].permute(3, 0, 1, 2, 4).reshape(NH, B * (S - 1), 4 * DH)                 # (NH, B*(S-1), 4*DH_out)
        dR = mm(a, b)
    if state0 is not None:   # step 0 pairs the initial h with dwx[0]
        a0 = state0[0].reshape(B, NH, DH).permute(1, 2, 0).to(dwx.dtype).contiguous()         # (NH, DH_in, B)
        b0 = dw[:, 0].permute(2, 0, 1, 3).reshape(NH, B, 4 * DH)                              # (NH, B, 4*DH_out)
        dR = dR + mm(a0, b0)
    db = dw.sum(dim=(0, 1), dtype=torch.float32).permute(1, 0, 2).contiguous()
    return dR.reshape(NH, DH, 4, DH), db


class SlstmFunction(torch.autograd.Function):
    """``slstm_forward`` with a backward pass: h, last = SlstmFunction.apply(wx, R, bias, state0)."""

    @staticmethod
    def forward(ctx, wx, R, bias, state0):
        h, last, cache = slstm_forward(wx, R, bias, state0, train_cache=True)
        ctx.save_for_backward(cache, R, h, state0 if state0 is not None else torch.empty(0, device=wx.device))
        ctx.has_state0 = state0 is not None
        ctx.dtypes = (wx.dtype, R.dtype, bias.dtype, None if state0 is None else state0.dtype)
        ctx.bias_shape = bias.shape
        return h, last

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, dh, dlast):
        cache, R, h, s0 = ctx.saved_tensors
        s0 = s0 if ctx.has_state0 else None
        if dh is None:
            dh = torch.zeros_like(h)
        dwx, ds0 = slstm_backward(cache, R, dh, dlast, s0)
        dR = db = None
        if ctx.needs_input_grad[1] or ctx.needs_input_grad[2]:
            dR, db = slstm_weight_grads(dwx, h, s0)
            dR = dR.to(ctx.dtypes[1])
            db = db.reshape(ctx.bias_shape).to(ctx.dtypes[2])
        return (dwx.to(ctx.dtypes[0]), dR, db, ds0.to(ctx.dtypes[3]) if ctx.has_state0 else None)


def add_rmsnorm(x, weight, y=None, eps: float = 1e-6, inplace: bool = False):
    """``x_new = x + y`` (when ``y`` is given) and ``RMSNorm(x_new) * weight`` in one pass; returns
    ``(x_new, normed)``.  This is the residual add of one sub-block fused with the pre-norm of the next
    (xlstm/xlstm_large/model.py:499-510; RMSNorm: components.py:70-97), with the reference's rounding points.
    ``x`` is (..., D) with contiguous rows; ``inplace`` writes ``x_new`` over ``x``."""
    _require_cuda(x, weight, y)
    if x.dtype not in _DTYPES or weight.dtype != x.dtype or (y is not None and (y.dtype != x.dtype or y.shape != x.shape)):
        raise ValueError("add_rmsnorm: x, y and weight must share one dtype (float32 or bfloat16) and x, y one shape")
    D = x.shape[-1]
    if weight.shape != (D,):
        raise ValueError("add_rmsnorm: weight must have shape (D,)")
    x2 = x.reshape(-1, D)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    y2 = None
    if y is not None:
        y2 = y.reshape(-1, D)
        if y2.stride(-1) != 1:
            y2 = y2.contiguous()
    normed = torch.empty((x2.shape[0], D), dtype=x.dtype, device=x.device)
    xo = None
    if y2 is not None:
        xo = x2 if (inplace and x2.data_ptr() == x.data_ptr()) else torch.empty((x2.shape[0], D), dtype=x.dtype, device=x.device)
    p = AddRmsnormParams()
    p.x, p.weight, p.normed = x2.data_ptr(), weight.contiguous().data_ptr(), normed.data_ptr()
    p.y = y2.data_ptr() if y2 is not None else None
    p.x_out = xo.data_ptr() if xo is not None else None
    p.rows, p.D = x2.shape[0], D
    p.x_sr, p.n_sr = x2.stride(0), D
    p.y_sr = y2.stride(0) if y2 is not None else 0
    p.xo_sr = xo.stride(0) if xo is not None else 0
    p.eps, p.dtype = eps, _DTYPES[x.dtype]
    with torch.cuda.device(x.device):
        check(lib().xl_add_rmsnorm(C.byref(p), _stream_ptr(x.device)), "xl_add_rmsnorm")
    x_new = x if xo is None else xo.reshape(x.shape)
    return x_new, normed.reshape(x.shape)


def headnorm_gate(h, o_preact, weight, eps: float = 1e-6):
    """``sigmoid(o_preact) * (LayerNorm over DH of h, per head) * weight`` -> (B, S, NH*DH).

    ``h`` is the cell output (B, NH, S, DH), read through its strides (no transpose copy); ``o_preact`` is
    (B, S, NH*DH), possibly a column slice of a wider projection output, or None: then the result is the plain
    per-head group norm ``(h - mean) * rstd * weight`` rounded once, the epilogue of the reference's sLSTM layer
    (``MultiHeadLayerNorm``, xlstm/components/ln.py:52-68; xlstm/blocks/slstm/layer.py:157).  Follows MultiHeadLayerNorm.forward
    and the output gate of the reference layer (components.py:188-242, xlstm_large/model.py:445-449)."""
    _require_cuda(h, o_preact, weight)
    if h.dim() != 4 or h.dtype not in _DTYPES or (o_preact is not None and o_preact.dtype != h.dtype) or weight.dtype != h.dtype:
        raise ValueError("headnorm_gate: h must be (B,NH,S,DH); h, o_preact and weight must share float32 or bfloat16")
    B, NH, S, DH = h.shape
    if (o_preact is not None and o_preact.shape != (B, S, NH * DH)) or weight.shape != (NH * DH,):
        raise ValueError("headnorm_gate: o_preact must be (B,S,NH*DH) and weight (NH*DH,)")
    h = _last_contig(h)
    o = _last_contig(o_preact) if o_preact is not None else None
    out = torch.empty((B, S, NH * DH), dtype=h.dtype, device=h.device)
    p = HeadnormGateParams()
    p.h, p.weight, p.out = h.data_ptr(), weight.contiguous().data_ptr(), out.data_ptr()
    p.B, p.NH, p.S, p.DH = B, NH, S, DH
    p.h_sb, p.h_sh, p.h_st = h.stride()[:3]
    if o is not None:
        p.o = o.data_ptr()
        p.o_sb, p.o_st = o.stride()[:2]
    p.eps, p.dtype = eps, _DTYPES[h.dtype]
    with torch.cuda.device(h.device):
        check(lib().xl_headnorm_gate(C.byref(p), _stream_ptr(h.device)), "xl_headnorm_gate")
    return out


def soft_cap(x, cap: float, out_float32: bool = False, float32_math: bool = False, bias=None):
    """``cap * tanh(x / cap)`` in one kernel with the rounding of the reference's eager ``soft_cap``
    (xlstm/xlstm_large/components.py:5-22).  ``out_float32`` returns the result (rounded to ``x.dtype``) as
    float32, the type the cell kernels take for gate pre-activations; with ``float32_math`` as well the
    quotient, tanh and product are not rounded to ``x.dtype`` in between (gates kept in fp32 in a bf16 model).
    ``x`` may be a column slice of a wider matrix (last dimension contiguous, one row stride); ``bias`` (last-dimension
    sized) is added first, which lets the gate projection ride in the q/k/v/o GEMM without its own launch."""
    if float32_math and not out_float32:
        raise ValueError("soft_cap: float32_math needs out_float32")
    _require_cuda(x, bias)
    if x.dtype not in _DTYPES:
        raise ValueError("soft_cap: float32 or bfloat16 only")
    cols = x.shape[-1]
    x2 = x.reshape(-1, cols) if x.dim() != 2 else x
    strided = x2.stride(-1) == 1 and x2.shape[0] > 0 and (x2.stride(0) != cols or bias is not None)
    if x2.stride(-1) != 1:
        x2, strided = x2.contiguous(), bias is not None
    out = torch.empty(x.shape, dtype=torch.float32 if out_float32 else x.dtype, device=x.device)
    p = SoftCapParams()
    p.x, p.out, p.n, p.cap = x2.data_ptr(), out.data_ptr(), x.numel(), float(cap)
    p.dtype, p.out_f32 = _DTYPES[x.dtype], (2 if float32_math else int(out_float32))
    if strided:
        p.cols, p.x_row_stride = cols, x2.stride(0)
        if bias is not None:
            if bias.shape != (cols,) or bias.dtype != x.dtype:
                raise ValueError("soft_cap: bias must have the size of the last dimension and x's dtype")
            p.bias = bias.contiguous().data_ptr()
    with torch.cuda.device(x.device):
        check(lib().xl_soft_cap(C.byref(p), _stream_ptr(x.device)), "xl_soft_cap")
    return out


def swiglu(gz):
    """``silu(gz[..., :F]) * gz[..., F:]`` in one kernel, the feed-forward's gating on the output of one projection that
    stacks ``proj_up_gate`` on ``proj_up`` (xlstm/xlstm_large/model.py:268-277), with the eager sequence's rounding."""
    _require_cuda(gz)
    if gz.dtype not in _DTYPES or gz.shape[-1] % 2:
        raise ValueError("swiglu: float32 or bfloat16, even last dimension")
    F_ = gz.shape[-1] // 2
    g2 = gz.reshape(-1, 2 * F_)
    if g2.stride(-1) != 1:
        g2 = g2.contiguous()
    out = torch.empty(gz.shape[:-1] + (F_,), dtype=gz.dtype, device=gz.device)
    p = SwigluParams()
    p.gz, p.out, p.rows, p.F, p.gz_row_stride, p.dtype = g2.data_ptr(), out.data_ptr(), g2.shape[0], F_, g2.stride(0), _DTYPES[gz.dtype]
    with torch.cuda.device(gz.device):
        check(lib().xl_swiglu(C.byref(p), _stream_ptr(gz.device)), "xl_swiglu")
    return out


def causal_conv1d(x, weight, bias=None, cu_seqlens=None, silu: bool = True):
    """Depthwise causal convolution over time and (by default) SiLU, the front of the reference's sLSTM layer
    (``CausalConv1d.forward``, xlstm/components/conv.py:110-129; activation xlstm/blocks/slstm/layer.py:133-142).

    x (B, S, F); weight (F, K) or the ``nn.Conv1d`` weight (F, 1, K); bias (F) or None.  With ``cu_seqlens`` (offsets on
    the flattened (B*S) axis) no tap reaches across a document boundary -- the reference's module knows rows only."""
    _require_cuda(x, weight, bias)
    if x.dim() != 3 or x.dtype not in _DTYPES:
        raise ValueError("causal_conv1d: x must be (B,S,F) in float32 or bfloat16")
    B, S, F_ = x.shape
    if weight.dim() == 3:
        weight = weight[:, 0, :]
    if weight.shape[0] != F_ or weight.dtype != x.dtype or (bias is not None and (bias.shape != (F_,) or bias.dtype != x.dtype)):
        raise ValueError("causal_conv1d: weight must be (F,K) and bias (F,), both in x's dtype")
    x = _last_contig(x)
    out = torch.empty((B, S, F_), dtype=x.dtype, device=x.device)
    p = Conv1dParams()
    w = weight.contiguous()
    p.x, p.weight, p.out = x.data_ptr(), w.data_ptr(), out.data_ptr()
    p.bias = bias.contiguous().data_ptr() if bias is not None else None
    nd = 0
    if cu_seqlens is not None:
        cu_dev, nd = prepare_cu_seqlens(cu_seqlens, B, S, x.device)
        p.cu_seqlens = cu_dev.data_ptr()
    p.B, p.S, p.F, p.K, p.num_docs, p.act = B, S, F_, w.shape[1], nd, int(bool(silu))
    p.x_sb, p.x_st = x.stride()[:2]
    p.o_sb, p.o_st = out.stride()[:2]
    p.dtype = _DTYPES[x.dtype]
    with torch.cuda.device(x.device):
        check(lib().xl_causal_conv1d(C.byref(p), _stream_ptr(x.device)), "xl_causal_conv1d")
    return out


def headwise_proj(inputs, weights, in_sel=None):
    """Up to four headwise (block-diagonal) projections in one launch, stacked in the sLSTM cell's input layout: the
    reference's ``LinearHeadwiseExpand.forward`` per gate (xlstm/components/linear_headwise.py:75-82, bias-free as the layer
    builds them) and the ``torch.cat`` of xlstm/blocks/slstm/layer.py:145-154.

    ``inputs``: one or two (..., NH*DH) bfloat16 tensors; ``weights``: list of (NH, DH, DH) parameters, slot order;
    ``in_sel[s]``: which input slot s projects (default: all the first).  Returns (..., len(weights) * NH * DH): slot-major,
    then head, then feature -- what the cell views as (.., 4, NH, DH)."""
    if isinstance(inputs, torch.Tensor):
        inputs = [inputs]
    inputs, weights = list(inputs), list(weights)
    n = len(weights)
    in_sel = [0] * n if in_sel is None else [int(i) for i in in_sel]
    _require_cuda(*inputs, *weights)
    if not (1 <= n <= 4) or not (1 <= len(inputs) <= 2) or len(in_sel) != n or any(i not in range(len(inputs)) for i in in_sel):
        raise ValueError("headwise_proj: one to four weights, one or two inputs, in_sel entries index the inputs")
    NH, DH, DH_in = weights[0].shape
    if DH != DH_in or DH not in (64, 128, 256):
        raise ValueError("headwise_proj: square per-head blocks of 64, 128 or 256 features only")
    D = NH * DH
    lead = inputs[0].shape[:-1]
    for x in inputs:
        if x.dtype != torch.bfloat16 or x.shape[-1] != D or x.shape[:-1] != lead:
            raise ValueError("headwise_proj: inputs must be bfloat16 (..., NH*DH) of one shape")
    for w in weights:
        if w.dtype != torch.bfloat16 or tuple(w.shape) != (NH, DH, DH):
            raise ValueError("headwise_proj: weights must be bfloat16 (NH, DH, DH)")
    xs = [_last_contig(x).reshape(-1, D) for x in inputs]
    xs = [x if x.stride(0) % 8 == 0 else x.contiguous() for x in xs]
    ws = [w.contiguous() for w in weights]
    rows = xs[0].shape[0]
    out = torch.empty((rows, n * D), dtype=torch.bfloat16, device=xs[0].device)
    p = HeadwiseParams()
    for i, x in enumerate(xs):
        p.x[i] = x.data_ptr()
        p.x_row_stride[i] = x.stride(0)
    for s_, w in enumerate(ws):
        p.w[s_] = w.data_ptr()
        p.in_sel[s_] = in_sel[s_]
    p.out, p.out_row_stride = out.data_ptr(), out.stride(0)
    dev = xs[0].device
    p.status = status_word(dev).data_ptr()
    p.rows, p.NH, p.DH, p.n_slots, p.dtype = rows, NH, DH, n, _DTYPES[torch.bfloat16]
    with torch.cuda.device(dev):
        check(lib().xl_headwise_proj(C.byref(p), _stream_ptr(dev)), "xl_headwise_proj")
    return out.reshape(*lead, n * D)


_greedy_scratch: dict[int, torch.Tensor] = {}


def softcap_argmax(logits, cap: float):
    """Greedy tokens of un-capped logits: ``argmax(soft_cap(logits, cap), dim=-1)`` with the reference's rounding and
    tie rule (xlstm/xlstm_large/model.py:149-151, generate.py:13-15) in one kernel.  ``logits`` is (..., V) with
    contiguous rows; returns int64 of shape ``logits.shape[:-1]``.  The kernel's scratch area is allocated once per
    device (and grown when more rows come) and shared by all calls on that device's streams in issue order."""
    _require_cuda(logits)
    if logits.dtype not in _DTYPES:
        raise ValueError("softcap_argmax: float32 or bfloat16 only")
    V = logits.shape[-1]
    x = logits.reshape(-1, V)
    if x.stride(-1) != 1:
        x = x.contiguous()
    rows = x.shape[0]
    dev = x.device
    need = int(lib().xl_softcap_argmax_scratch_bytes(rows))
    sc = _greedy_scratch.get(dev.index)
    if sc is None or sc.numel() < need:
        sc = torch.zeros(max(need, int(lib().xl_softcap_argmax_scratch_bytes(256))), dtype=torch.uint8, device=dev)
        _greedy_scratch[dev.index] = sc
    out = torch.empty(rows, dtype=torch.int64, device=dev)
    p = GreedyParams()
    p.logits, p.tokens, p.scratch, p.scratch_bytes = x.data_ptr(), out.data_ptr(), sc.data_ptr(), sc.numel()
    p.rows, p.V, p.row_stride, p.cap, p.dtype = rows, V, x.stride(0), float(cap), _DTYPES[x.dtype]
    with torch.cuda.device(dev):
        check(lib().xl_softcap_argmax(C.byref(p), _stream_ptr(dev)), "xl_softcap_argmax")
    return out.reshape(logits.shape[:-1])
