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


# ------------------------------------------------------------------------------------------ backward through time
def _grads_oracle(wx, R, bias, st, gh, gl, stabiliser_grad):
    wx_o, R_o, b_o = wx.float().requires_grad_(), R.float().requires_grad_(), bias.clone().requires_grad_()
    s_o = None if st is None else st.clone().requires_grad_()
    h, last = O.slstm_forward(wx_o, R_o, b_o, s_o, stabiliser_grad=stabiliser_grad)
    ((h * gh.float()).sum() + (last * gl).sum()).backward()
    return h.detach(), wx_o.grad, R_o.grad, b_o.grad, (None if s_o is None else s_o.grad)


def _grads_kernel(wx, R, bias, st, gh, gl):
    import xlstm_b200
    from xlstm_b200 import ops
    wx_k, R_k, b_k = wx.cuda().requires_grad_(), R.cuda().requires_grad_(), bias.cuda().requires_grad_()
    s_k = None if st is None else st.cuda().requires_grad_()
    h, last = ops.SlstmFunction.apply(wx_k, R_k, b_k, s_k)
    ((h.float() * gh.cuda().float()).sum() + (last * gl.cuda()).sum()).backward()
    xlstm_b200.check_device_status()
    return (h.detach().float().cpu(), wx_k.grad.float().cpu(), R_k.grad.float().cpu(), b_k.grad.float().cpu(),
            None if s_k is None else s_k.grad.cpu())


@pytest.mark.parametrize("B,S,NH,DH,with_state,state_loss", [
    (2, 1, 1, 64, True, False), (2, 2, 2, 64, False, False), (1, 9, 1, 128, True, True),
    (3, 5, 1, 64, False, False), (3, 37, 2, 64, True, False), (16, 64, 4, 256, True, False),
    (20, 33, 1, 128, True, True), (16, 200, 2, 256, False, True)])
def test_backward_matches_autograd_of_the_oracle(B, S, NH, DH, with_state, state_loss):
    """dWx, dR, dbias and the gradient of the initial state from the backward kernel against autograd over the CPU
    oracle on the same bf16-rounded inputs.  With a loss on the final c and n as well (``state_loss``) the oracle holds
    the stabiliser constant, which is the reference kernel's rule (slstm_pointwise.cu:118-196); m itself never gets a
    gradient.  Tolerance: relative L2 <= 1e-2 (gates and h are cached in bf16, dWx leaves in bf16)."""
    wx, R, bias, st = _case(B * 100 + S + 1, B, S, NH, DH, with_state)
    g = torch.Generator().manual_seed(3)
    gh = torch.randn(B, NH, S, DH, generator=g).bfloat16()
    gl = torch.randn(4, B, NH * DH, generator=g)
    if not state_loss:
        gl[1:] = 0
    gl[3] = 0
    ref = _grads_oracle(wx, R, bias, st, gh, gl, stabiliser_grad=not state_loss)
    got = _grads_kernel(wx, R, bias, st, gh, gl)
    for name, a, b in zip(("h", "dwx", "dR", "dbias"), got[:4], ref[:4]):
        assert torch.isfinite(a).all(), name
        assert rel_l2(a, b) < TOL, (name, rel_l2(a, b))
    if with_state:
        for idx in range(3):
            assert rel_l2(got[4][idx], ref[4][idx]) < TOL, (idx, rel_l2(got[4][idx], ref[4][idx]))
        assert float(got[4][3].abs().max()) == 0.0  # the stabiliser gets no gradient


def test_backward_matches_reference_vanilla_gradient_fixture():
    """The gradients autograd gives over the reference's own vanilla cell (fp32, DH = 64), reproduced by the kernels on
    the bf16-rounded inputs."""
    g = load_golden("slstm_grad_state")
    wx, R = g["wx"].bfloat16(), g["R"].bfloat16()
    gl = torch.zeros(4, *g["gl"].shape)
    gl[0] = g["gl"]
    got = _grads_kernel(wx, R, g["bias"], g["state0"], g["gh"].bfloat16(), gl)
    assert rel_l2(got[0], g["out"]) < TOL
    for name, a, b in zip(("dwx", "dR", "dbias"), got[1:4], (g["dwx"], g["dR"], g["dbias"])):
        assert rel_l2(a, b) < 2e-2, (name, rel_l2(a, b))  # the fixture is fp32 on unrounded inputs
    for idx in range(3):
        assert rel_l2(got[4][idx], g["dstate0"][idx]) < 2e-2


def test_training_forward_equals_inference_forward_and_long_backward_is_finite():
    """The cache-writing forward gives bit-identical h and final state; 2048 steps back through the block-stack
    benchmark's cell (B=16, NH=4, DH=256) stay finite and agree with the oracle on the last 64 steps' dWx (whose
    gradient does not depend on earlier steps' caches)."""
    import xlstm_b200
    from xlstm_b200 import ops
    wx, R, bias, _ = _case(9, 16, 2048, 4, 256)
    out, last = xlstm_b200.slstm_forward(wx.cuda(), R.cuda(), bias.cuda())
    out_t, last_t, cache = ops.slstm_forward(wx.cuda(), R.cuda(), bias.cuda(), train_cache=True)
    assert torch.equal(out, out_t) and torch.equal(last, last_t)
    g = torch.Generator().manual_seed(4)
    gh = torch.randn(16, 4, 2048, 256, generator=g).bfloat16()
    dwx, ds0 = ops.slstm_backward(cache, R.cuda(), gh.cuda())
    xlstm_b200.check_device_status()
    assert torch.isfinite(dwx).all() and torch.isfinite(ds0).all()
    # oracle on the tail: start it from the kernel's own state at step 2048 - 64 (taken from a shorter forward)
    T = 64
    _, mid = xlstm_b200.slstm_forward(wx[:, :-T].cuda(), R.cuda(), bias.cuda())
    wx_o = wx[:, -T:].float().requires_grad_()
    h_o, _ = O.slstm_forward(wx_o, R.float(), bias, mid.cpu())
    (h_o * gh[:, :, -T:].float()).sum().backward()
    assert rel_l2(dwx[:, -T:].float().cpu(), wx_o.grad) < TOL


def test_forward_and_backward_are_bit_identical_from_run_to_run():
    """Partial sums cross the cluster through double-buffered tiles and are added in rank order: repeated runs must
    agree to the last bit (a race on one of the alternating buffers would show up here).  Three batch groups with a
    ragged last one, three heads."""
    import xlstm_b200
    from xlstm_b200 import ops
    wx, R, bias, _ = _case(10, 37, 300, 3, 128)
    gh = torch.randn(37, 3, 300, 128, generator=torch.Generator().manual_seed(5)).bfloat16().cuda()
    wx, R, bias = wx.cuda(), R.cuda(), bias.cuda()
    first = None
    for _ in range(6):
        h, last, cache = ops.slstm_forward(wx, R, bias, train_cache=True)
        dwx, ds0 = ops.slstm_backward(cache, R, gh)
        cur = (h, last, dwx, ds0)
        if first is None:
            first = cur
        else:
            assert all(torch.equal(a, b) for a, b in zip(first, cur))
    xlstm_b200.check_device_status()
