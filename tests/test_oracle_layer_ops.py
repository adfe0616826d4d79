"""The CPU oracle of the cell-adjacent operators against fixtures produced by the reference's own norm modules."""
import pytest
import torch

from conftest import load_golden, rel_l2
from oracle import layer_ops as O

DT = {"f32": torch.float32, "bf16": torch.bfloat16}


@pytest.mark.parametrize("tag", ["f32", "bf16"])
def test_add_rmsnorm_matches_reference_modules(tag):
    g, dt = load_golden("layer_ops"), DT[tag]
    x, y, w = (g[f"rms_{tag}_{k}"].to(dt) for k in ("x", "y", "w"))
    x_new, normed = O.add_rmsnorm(x, w, y, eps=1e-6)
    # the same rounding points as the eager reference: bit-exact in bf16, reduction order only in fp32
    assert torch.equal(x_new.float(), g[f"rms_{tag}_xnew"])
    tol = 0.0 if tag == "bf16" else 1e-6
    assert (normed.float() - g[f"rms_{tag}_normed"]).abs().max().item() <= tol


@pytest.mark.parametrize("tag", ["f32", "bf16"])
def test_headnorm_gate_matches_reference_modules(tag):
    g, dt = load_golden("layer_ops"), DT[tag]
    h, o, w = (g[f"hng_{tag}_{k}"].to(dt) for k in ("h", "o", "w"))
    out = O.headnorm_gate(h, o, w, eps=1e-6)
    tol = 0.0 if tag == "bf16" else 1e-6
    assert (out.float() - g[f"hng_{tag}_out"]).abs().max().item() <= tol


def test_add_rmsnorm_without_residual_returns_input():
    x = torch.randn(3, 64)
    x_new, normed = O.add_rmsnorm(x, torch.ones(64))
    assert x_new is x
    assert torch.allclose(normed.pow(2).mean(-1), torch.ones(3), atol=1e-4)


@pytest.mark.parametrize("tag", ["f32", "bf16"])
def test_soft_cap_matches_reference_function(tag):
    g, dt = load_golden("layer_ops"), DT[tag]
    x = g[f"cap_{tag}_x"].to(dt)
    for cap in (15.0, 30.0):
        want = g[f"cap_{tag}_{int(cap)}"]
        got = O.soft_cap(x, cap)
        tol = 0.0 if tag == "bf16" else 4e-6
        assert (got.float() - want).abs().max().item() <= tol
        assert torch.equal(O.soft_cap(x, cap, out_float32=True), got.float())


@pytest.mark.parametrize("tag", ["f32", "bf16"])
def test_causal_conv1d_matches_reference_module(tag):
    """Rows, and rows packed from documents (the reference module run once per document)."""
    g, dt = load_golden("conv"), DT[tag]
    x, w, b = (g[f"{tag}_{k}"].to(dt) for k in "xwb")
    tol = 0.0 if tag == "bf16" else 4e-6
    assert (O.causal_conv1d(x, w, b).float() - g[f"{tag}_rows"]).abs().max().item() <= tol
    packed = O.causal_conv1d(x, w, b, cu_seqlens=g["cu"].tolist())
    assert (packed.float() - g[f"{tag}_packed"]).abs().max().item() <= tol
    # the fixture itself shows why the offsets matter: without them the taps reach into the previous document
    assert (g[f"{tag}_rows"] - g[f"{tag}_packed"]).abs().max().item() > 1.0


@pytest.mark.parametrize("tag", ["a", "b"])
def test_headwise_proj_matches_reference_modules(tag):
    """Four ``LinearHeadwiseExpand`` modules of the reference, used as its sLSTM layer uses them, and the concatenation."""
    g = load_golden("headwise")
    bf = lambda t: t.view(torch.bfloat16)
    x, xc, want = bf(g[f"{tag}_x"]), bf(g[f"{tag}_xc"]), bf(g[f"{tag}_y"]).float()
    got = O.headwise_proj([x, xc], [bf(g[f"{tag}_w{i}"]) for i in range(4)], [1, 1, 0, 0]).float()
    d = (got - want).abs()
    assert (d > 0).float().mean().item() < 1e-3 and rel_l2(got, want) < 1e-6   # the summation order may move a last bit
