"""The sLSTM CPU oracle against fixtures produced by the reference's vanilla cell."""
import pytest
import torch

from conftest import load_golden, rel_l2
from oracle import slstm as O


@pytest.mark.parametrize("name", ["slstm_zero", "slstm_state", "slstm_b1s1"])
def test_matches_reference_vanilla_fp32(name):
    g = load_golden(name)
    # the fixtures have either all rows fresh or none, where both "fresh" rules coincide
    for rule in ("elementwise", "whole_tensor"):
        out, last = O.slstm_forward(g["wx"], g["R"], g["bias"], g.get("state0"), fresh_rule=rule)
        assert rel_l2(out, g["out"]) < 1e-5
        assert rel_l2(last, g["last"]) < 1e-5


def test_matches_reference_vanilla_bf16_states():
    g = load_golden("slstm_bf16")
    out, last = O.slstm_forward(g["wx"], g["R"], g["bias"], state_dtype=torch.bfloat16)
    # the reference ran every op in bf16; the oracle runs fp32 math and rounds the states to bf16 each step
    assert rel_l2(out, g["out"]) < 2e-2
    assert rel_l2(last[0], g["last"][0]) < 2e-2


def test_reset_equals_separate_documents():
    torch.manual_seed(1)
    B, S, NH, DH = 2, 12, 2, 8
    H = NH * DH
    wx = torch.randn(B, S, 4 * H)
    R = torch.randn(NH, DH, 4, DH) * 0.2
    bias = torch.randn(NH, 4, DH) * 0.1
    reset = torch.zeros(B, S, dtype=torch.bool)
    reset[0, 5] = True
    out, last = O.slstm_forward(wx, R, bias, reset=reset)
    a, _ = O.slstm_forward(wx[:1, :5], R, bias)
    b, lb = O.slstm_forward(wx[:1, 5:], R, bias)
    assert rel_l2(out[0, :, :5], a[0]) < 1e-6
    assert rel_l2(out[0, :, 5:], b[0]) < 1e-6
    assert rel_l2(last[:, 0], lb[:, 0]) < 1e-6


@pytest.mark.parametrize("name", ["slstm_grad", "slstm_grad_state"])
@pytest.mark.parametrize("stabiliser_grad", [True, False])
def test_autograd_of_the_oracle_matches_reference_vanilla_gradients(name, stabiliser_grad):
    """Autograd over the oracle is the oracle of the backward kernel: it reproduces the gradients autograd gives over
    the reference's vanilla cell, with the stabiliser differentiated or held constant (the loss reads h only)."""
    g = load_golden(name)
    wx = g["wx"].clone().requires_grad_()
    R = g["R"].clone().requires_grad_()
    bias = g["bias"].clone().requires_grad_()
    s0 = g["state0"].clone().requires_grad_() if "state0" in g else None
    out, last = O.slstm_forward(wx, R, bias, s0, stabiliser_grad=stabiliser_grad)
    assert rel_l2(out.detach(), g["out"]) < 1e-5
    ((out * g["gh"]).sum() + (last[0] * g["gl"]).sum()).backward()
    assert rel_l2(wx.grad, g["dwx"]) < 1e-4
    assert rel_l2(R.grad, g["dR"]) < 1e-4
    assert rel_l2(bias.grad, g["dbias"]) < 1e-4
    if s0 is not None:
        for i in range(3):  # h, c, n; the stabiliser's own gradient is a matter of convention
            assert rel_l2(s0.grad[i], g["dstate0"][i]) < 1e-4
