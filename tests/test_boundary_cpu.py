"""Host-side checks that need no GPU: the C-ABI library loads and exports what the header declares,
argument validation, and the drop-in boundary against the reference checkout when it is present."""
import ctypes
import os
import re
import sys

import pytest
import torch

from conftest import ROOT, import_reference, rel_l2


def test_library_exports_every_declared_symbol():
    from xlstm_b200 import _lib
    header = open(os.path.join(ROOT, "include", "xlstm_b200.h")).read()
    declared = set(re.findall(r"\b(xl_[a-z_0-9]+)\s*\(", header))
    assert declared == set(_lib.EXPORTS)
    l = _lib.lib()
    for name in declared:
        assert hasattr(l, name), name
    assert l.xl_abi_version() == 3
    assert b"stride" in l.xl_strerror(-3)


def test_struct_layouts_match_header_field_order():
    from xlstm_b200 import _lib
    header = open(os.path.join(ROOT, "include", "xlstm_b200.h")).read()
    for cname, struct in (("xl_mlstm_seq_params", _lib.MlstmSeqParams), ("xl_mlstm_step_params", _lib.MlstmStepParams),
                          ("xl_slstm_params", _lib.SlstmParams), ("xl_add_rmsnorm_params", _lib.AddRmsnormParams),
                          ("xl_headnorm_gate_params", _lib.HeadnormGateParams), ("xl_soft_cap_params", _lib.SoftCapParams),
                          ("xl_conv1d_params", _lib.Conv1dParams), ("xl_greedy_params", _lib.GreedyParams),
                          ("xl_swiglu_params", _lib.SwigluParams), ("xl_peer_reduce_params", _lib.PeerReduceParams),
                          ("xl_headwise_params", _lib.HeadwiseParams), ("xl_mlstm_decode_cell_params", _lib.MlstmDecodeCellParams),
                          ("xl_slstm_bwd_params", _lib.SlstmBwdParams)):
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (cname, cname), header, re.S).group(1)
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        body = re.sub(r"\[\d+\]", "", body)   # array members: the name is what counts
        names = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            first, *rest = decl.split(",")
            names.append(re.findall(r"[A-Za-z_0-9]+", first)[-1])
            names += [re.findall(r"[A-Za-z_0-9]+", r)[-1] for r in rest]
        assert names == [f[0] for f in struct._fields_], cname


def test_entry_points_validate_before_launching():
    from xlstm_b200 import _lib
    l = _lib.lib()
    p = _lib.MlstmSeqParams()
    assert l.xl_mlstm_chunkwise(ctypes.byref(p), None) == -1  # null pointers
    assert l.xl_mlstm_recurrent(ctypes.byref(p), None) == -1
    sp = _lib.MlstmStepParams()
    assert l.xl_mlstm_step(ctypes.byref(sp), None) == -1
    sl = _lib.SlstmParams()
    assert l.xl_slstm_forward(ctypes.byref(sl), None) == -1
    # fake but non-null pointers: shape / dtype checks fire, nothing is launched
    for name in ("q", "k", "v", "h", "igate", "fgate", "c_out", "n_out", "m_out"):
        setattr(p, name, 0x1000)
    assert l.xl_mlstm_chunkwise(ctypes.byref(p), None) == -2
    p.B, p.NH, p.S, p.DHQK, p.DHV, p.dtype = 1, 1, 64, 96, 128, 1
    assert l.xl_mlstm_chunkwise(ctypes.byref(p), None) == -6  # DHQK not covered by the tensor-core kernel
    p.DHQK = 64
    p.q_st = p.k_st = p.v_st = 100  # not a multiple of 8 elements
    assert l.xl_mlstm_chunkwise(ctypes.byref(p), None) == -3
    p.c0, p.n0, p.m0 = 0x2000, p.n_out, 0x3000
    assert l.xl_mlstm_recurrent(ctypes.byref(p), None) == -9  # n_out aliases n0


def test_newer_entry_points_validate_before_launching():
    from xlstm_b200 import _lib
    l = _lib.lib()
    hw = _lib.HeadwiseParams()
    assert l.xl_headwise_proj(ctypes.byref(hw), None) == -1          # null pointers
    hw.x[0], hw.out, hw.w[0] = 0x1000, 0x2000, 0x3000
    hw.dtype, hw.n_slots, hw.NH, hw.DH, hw.rows = 1, 1, 2, 96, 4
    assert l.xl_headwise_proj(ctypes.byref(hw), None) == -6          # block size not covered
    hw.DH, hw.n_slots = 64, 5
    assert l.xl_headwise_proj(ctypes.byref(hw), None) == -2          # more than four slots
    hw.n_slots, hw.dtype = 1, 0
    assert l.xl_headwise_proj(ctypes.byref(hw), None) == -5          # bf16 only
    hw.dtype = 1
    hw.x_row_stride[0], hw.out_row_stride = 100, 128
    assert l.xl_headwise_proj(ctypes.byref(hw), None) == -3          # row stride below NH * DH
    dc = _lib.MlstmDecodeCellParams()
    assert l.xl_mlstm_decode_cell(ctypes.byref(dc), None) == -1
    for name in ("q", "k", "v", "c_out", "n_out", "m_out"):
        setattr(dc.step, name, 0x1000)
    dc.step.B, dc.step.NH, dc.step.DHQK, dc.step.DHV, dc.step.dtype = 2, 2, 64, 128, 1
    assert l.xl_mlstm_decode_cell(ctypes.byref(dc), None) == -1      # the fused operands are missing
    dc.gates_raw = dc.ogate = dc.norm_weight = dc.hg = 0x2000
    dc.gate_cap = 15.0
    dc.step.DHV = 2048
    assert l.xl_mlstm_decode_cell(ctypes.byref(dc), None) == -6      # more than eight blocks per head
    dc.step.DHV = 128
    dc.gr_sb, dc.o_sb, dc.hg_sb = 2, 256, 256
    assert l.xl_mlstm_decode_cell(ctypes.byref(dc), None) == -3      # gate rows shorter than 2 * NH
    sb = _lib.SlstmBwdParams()
    assert l.xl_slstm_backward(ctypes.byref(sb), None) == -1         # null pointers
    sb.cache = sb.R = sb.dh = sb.dwx = sb.dstate0 = 0x1000
    sb.B, sb.S, sb.NH, sb.DH, sb.dtype = 2, 3, 2, 64, 0
    assert l.xl_slstm_backward(ctypes.byref(sb), None) == -5         # bf16 only
    sb.dtype, sb.DH = 1, 96
    assert l.xl_slstm_backward(ctypes.byref(sb), None) == -6         # head size not covered
    sb.DH, sb.dwx = 64, 0x1008
    assert l.xl_slstm_backward(ctypes.byref(sb), None) == -4         # dwx leaves in 16-byte pieces
    assert l.xl_slstm_cache_bytes(16, 2048, 4, 256) == 32 * 2048 * 128 * 96
    assert l.xl_slstm_cache_bytes(17, 1, 1, 64) == 2 * 2 * 128 * 96   # two 16-row groups, two CTAs per cluster
    assert l.xl_slstm_cache_bytes(4, 4, 1, 48) == 0
    sl = _lib.SlstmParams()
    sl.wx = sl.R = sl.bias = sl.h_out = sl.state_out = 0x1000
    sl.B, sl.S, sl.NH, sl.DH, sl.dtype = 2, 3, 2, 64, 1
    sl.train_cache, sl.cu_seqlens, sl.num_docs = 0x2000, 0x3000, 1
    assert l.xl_slstm_forward(ctypes.byref(sl), None) == -6          # no training cache with document offsets


def test_ops_refuse_cpu_tensors():
    import xlstm_b200
    q = torch.zeros(1, 1, 64, 64)
    with pytest.raises(ValueError, match="no CPU path"):
        xlstm_b200.mlstm_sequence(q, q, q, torch.zeros(1, 1, 64), torch.zeros(1, 1, 64))


def test_cu_seqlens_validation():
    from xlstm_b200.ops import prepare_cu_seqlens
    with pytest.raises(ValueError):
        prepare_cu_seqlens([0, 5, 3, 16], 2, 8, "cpu")
    with pytest.raises(ValueError):
        prepare_cu_seqlens([0, 5, 12, 16], 2, 8, "cpu")  # straddles the row boundary at 8
    with pytest.raises(ValueError):
        prepare_cu_seqlens([0, 8], 2, 8, "cpu")
    cu, nd = prepare_cu_seqlens([0, 3, 3, 8, 16], 2, 8, "cpu")
    assert nd == 4 and cu.dtype == torch.int32


def _register_native_oracle():
    """The upstream 'native' kernel names, served by the CPU oracle (test infrastructure only)."""
    from oracle import mlstm as O
    from xlstm_b200 import backend_module as bm

    def chunk(q, k, v, i, f, c_initial=None, n_initial=None, m_initial=None, chunk_size=64, eps=1e-6, **_):
        h, st = O.mlstm_chunkwise(q, k, v, i, f, c_initial, n_initial, m_initial, chunk_size=chunk_size, eps=eps)
        return h.to(q.dtype), st

    def seq(q, k, v, i, f, c_initial=None, n_initial=None, m_initial=None, eps=1e-6, **_):
        h, st = O.mlstm_sequence(q, k, v, i, f, c_initial, n_initial, m_initial, eps=eps)
        return h.to(q.dtype), st

    def step(q, k, v, i, f, c=None, n=None, m=None, eps=1e-6, **_):
        h, st = O.mlstm_step(q, k, v, i, f, c, n, m, eps=eps)
        return h.to(q.dtype), st

    bm.register_kernel("chunkwise", "chunkwise--native_autograd", chunk)
    bm.register_kernel("sequence", "native_sequence__native", seq)
    bm.register_kernel("step", "native", step)


def test_reference_model_runs_unchanged_on_the_shim():
    """The reference's small test model: its xlstm_large/model.py imports the shim, builds with
    the native triple (served by the oracle) and with the b200 names, and chunkwise == step-by-step."""
    import_reference()
    _register_native_oracle()
    from xlstm.xlstm_large.model import xLSTMLarge, xLSTMLargeConfig
    torch.manual_seed(0)
    cfg = xLSTMLargeConfig(embedding_dim=128, num_heads=4, num_blocks=2, vocab_size=256, return_last_states=True,
                           mode="inference", chunkwise_kernel="chunkwise--native_autograd",
                           sequence_kernel="native_sequence__native", step_kernel="native")
    model = xLSTMLarge(cfg).eval()
    x = torch.randint(0, 256, (2, 150))
    with torch.no_grad():
        logits, state = model(x)
        assert logits.shape == (2, 150, 256) and len(state) == 2 and len(state[0]) == 3
        # token-by-token through the step kernel (tests/template_chunkwise_vs_recurrent.py in the reference)
        st = None
        outs = []
        for t in range(150):
            lg, st = model(x[:, t:t + 1], st)
            outs.append(lg)
    torch.testing.assert_close(torch.cat(outs, 1), logits, atol=4e-3, rtol=5e-2)
    # construction with the CUDA kernel names goes through the same selectors
    cfg2 = xLSTMLargeConfig(embedding_dim=128, num_heads=4, num_blocks=1, vocab_size=64, mode="inference",
                            chunkwise_kernel="chunkwise--b200", sequence_kernel="native_sequence__b200", step_kernel="b200")
    xLSTMLarge(cfg2)
    with pytest.raises(ValueError):
        xLSTMLarge(xLSTMLargeConfig(embedding_dim=128, num_heads=4, num_blocks=1, vocab_size=64, step_kernel="nope"))


def test_reference_slstm_switch_accepts_b200():
    import_reference()
    from xlstm_b200.integration import install_slstm_backend
    cls = install_slstm_backend()
    from xlstm.blocks.slstm.cell import sLSTMCell, sLSTMCellConfig
    cell = sLSTMCell(sLSTMCellConfig(hidden_size=128, num_heads=2, backend="b200", recurrent_weight_init="standard"))
    assert isinstance(cell, cls)
    assert cell._recurrent_kernel_.shape == (2, 64, 4, 64) and cell._bias_.shape == (2, 4, 64)
    van = sLSTMCell(sLSTMCellConfig(hidden_size=128, num_heads=2, backend="vanilla"))
    assert type(van).__name__ == "sLSTMCell_vanilla"
    with pytest.raises(ValueError, match="no CPU path"):
        cell(torch.zeros(1, 4, 512, dtype=torch.bfloat16))
    # the whole block stack builds with the new backend name
    from xlstm.xlstm_block_stack import xLSTMBlockStack, xLSTMBlockStackConfig
    from xlstm.blocks.slstm.block import sLSTMBlockConfig
    from xlstm.blocks.slstm.layer import sLSTMLayerConfig
    cfg = xLSTMBlockStackConfig(slstm_block=sLSTMBlockConfig(slstm=sLSTMLayerConfig(num_heads=2, conv1d_kernel_size=4, backend="b200")),
                                num_blocks=2, embedding_dim=128, slstm_at="all")
    xLSTMBlockStack(cfg)


def test_slstm_weight_grads_equal_autograd_over_the_oracle():
    """dR and dbias are sums over (b,t) of h_{t-1} (x) dWx_t and dWx_t (host-side matrix products over the backward
    kernel's output): with dWx and h taken from the oracle they must reproduce autograd's gradients of R and the bias,
    the initial h included."""
    from oracle import slstm as O
    from xlstm_b200 import ops
    from conftest import rel_l2
    torch.manual_seed(0)
    B, S, NH, DH = 3, 11, 2, 8
    H = NH * DH
    for with_state in (True, False):
        wx = torch.randn(B, S, 4 * H, requires_grad=True)
        R = (torch.randn(NH, DH, 4, DH) * 0.3).requires_grad_()
        bias = torch.randn(NH, 4, DH, requires_grad=True)
        s0 = None
        if with_state:
            s0 = torch.randn(4, B, H)
            s0[2] = s0[2].abs() + 0.5
        h, _ = O.slstm_forward(wx, R, bias, s0)
        (h * torch.randn_like(h)).sum().backward()
        dR, db = ops.slstm_weight_grads(wx.grad, h.detach(), s0)
        assert rel_l2(dR, R.grad) < 1e-5 and rel_l2(db, bias.grad) < 1e-5
    # a single step: only the initial h contributes
    dR1, _ = ops.slstm_weight_grads(wx.grad[:, :1], h.detach()[:, :, :1], None)
    assert float(dR1.abs().max()) == 0.0
