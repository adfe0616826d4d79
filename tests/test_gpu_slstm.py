"""Parity of the persistent sLSTM kernel (through the C ABI) with the CPU oracle and the reference fixture."""
import pytest
import torch

from conftest import load_golden, rel_l2
from oracle import slstm as O

pytestmark = pytest.mark.gpu
TOL = 1e-2  # relative L2 on bf16 outputs and final states


def _case(seed, B, S, NH, DH, with_state=False):
    g = torch.Generator().manual_seed(seed)
    H = NH * DH
    wx = torch.randn(B, S, 4 * H, generator=g).bfloat16()
    R = ((torch.rand(NH, DH, 4, DH, generator=g) * 2 - 1) / H ** 0.5).bfloat16()
    bias = torch.randn(NH, 4, DH, generator=g) * 0.5
    st = None
    if with_state:
        st = torch.randn(4, B, H, generator=g)
        st[2] = st[2].abs() + 0.5
        st[0] = st[0].bfloat16().float()
    return wx, R, bias, st


def _run(wx, R, bias, st=None, cu=None):
    import xlstm_b200
    out, last = xlstm_b200.slstm_forward(wx.cuda(), R.cuda(), bias.cuda(), None if st is None else st.cuda(), cu_seqlens=cu)
    xlstm_b200.check_device_status()
    return out.float().cpu(), last.cpu()


@pytest.mark.parametrize("B,S,NH,DH,with_state", [(16, 64, 4, 256, False), (3, 37, 2, 64, True), (20, 16, 1, 128, False),
                                                  (1, 1, 4, 64, False)])
def test_matches_oracle(B, S, NH, DH, with_state):
    wx, R, bias, st = _case(B * 100 + S, B, S, NH, DH, with_state)
    out_ref, last_ref = O.slstm_forward(wx, R, bias, st)
    out, last = _run(wx, R, bias, st)
    assert torch.isfinite(out).all()
    assert rel_l2(out, out_ref) < TOL, rel_l2(out, out_ref)
    for idx in range(4):
        assert rel_l2(last[idx], last_ref[idx]) < TOL, (idx, rel_l2(last[idx], last_ref[idx]))


def test_matches_reference_vanilla_fixture():
    g = load_golden("slstm_bf16")  # produced by the reference's vanilla cell in bf16
    out, last = _run(g["wx"].bfloat16(), g["R"].bfloat16(), g["bias"])
    assert rel_l2(out, g["out"]) < 2e-2  # the fixture itself carries bf16 state rounding
    out32, _ = O.slstm_forward(g["wx"], g["R"], g["bias"])
    assert rel_l2(out, out32) < TOL


def test_document_boundaries_reset_state_in_kernel():
    B, S, NH, DH = 3, 48, 2, 64
    wx, R, bias, _ = _case(5, B, S, NH, DH)
    cu = [0, 7, 7, 48, 48 + 20, 96, 96 + 48]
    reset = torch.zeros(B, S, dtype=torch.bool)
    reset[0, 7] = True
    reset[1, 20] = True
    out_ref, last_ref = O.slstm_forward(wx, R, bias, reset=reset)
    out, last = _run(wx, R, bias, cu=cu)
    assert rel_l2(out, out_ref) < TOL and rel_l2(last, last_ref) < TOL


def test_long_sequence_stays_in_tolerance():
    """Config-3 cell shape (B=16, NH=4, DH=256) over 512 steps: error must not accumulate past the budget."""
    wx, R, bias, _ = _case(6, 16, 512, 4, 256)
    out_ref, last_ref = O.slstm_forward(wx, R, bias)
    out, last = _run(wx, R, bias)
    assert rel_l2(out, out_ref) < TOL and rel_l2(last[1], last_ref[1]) < TOL


def test_full_length_sequence_2048_steps_against_the_oracle():
    """The block-stack benchmark's cell shape at its full length: B=16, NH=4, DH=256, S=2048.  The kernel uses the
    hardware exponential, logarithm and reciprocal throughout; 2048 steps must not accumulate their error."""
    wx, R, bias, _ = _case(8, 16, 2048, 4, 256)
    out_ref, last_ref = O.slstm_forward(wx, R, bias)
    out, last = _run(wx, R, bias)
    assert torch.isfinite(out).all()
    assert rel_l2(out, out_ref) < TOL, rel_l2(out, out_ref)
    assert rel_l2(out[:, :, -256:], out_ref[:, :, -256:]) < TOL
    for idx in range(4):
        assert rel_l2(last[idx], last_ref[idx]) < TOL, (idx, rel_l2(last[idx], last_ref[idx]))
