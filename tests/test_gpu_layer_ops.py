"""Parity of the cell-adjacent kernels (through the C ABI) with the CPU oracle and the reference-module fixtures.

Tolerances: the kernels round where the reference's eager operators round, so bf16 results may differ from the
oracle only where the fp32 reduction order moves a value across a rounding boundary: at most one bf16 step
(relative 2^-7) on under 1 % of the elements.  fp32 results agree to 2e-6 relative to the row scale."""
import pytest
import torch

from conftest import load_golden, rel_l2
from oracle import layer_ops as O

pytestmark = pytest.mark.gpu
DT = {"f32": torch.float32, "bf16": torch.bfloat16}


def _close(got, want, dt):
    got, want = got.float().cpu(), want.float().cpu()
    diff = (got - want).abs()
    if dt == torch.bfloat16:
        assert (diff <= want.abs() * 2.0 ** -7 + 1e-30).all(), float(diff.max())
        assert (diff == 0).float().mean().item() > 0.99
    else:
        assert float(diff.max()) <= 2e-6 * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("tag", ["f32", "bf16"])
def test_kernels_match_reference_module_fixtures(tag):
    import xlstm_b200
    g, dt = load_golden("layer_ops"), DT[tag]
    x, y, w = (g[f"rms_{tag}_{k}"].to(dt).cuda() for k in ("x", "y", "w"))
    x_new, normed = xlstm_b200.add_rmsnorm(x, w, y, eps=1e-6)
    assert torch.equal(x_new.float().cpu(), g[f"rms_{tag}_xnew"])
    _close(normed, g[f"rms_{tag}_normed"], dt)
    h, o, w2 = (g[f"hng_{tag}_{k}"].to(dt).cuda() for k in ("h", "o", "w"))
    _close(xlstm_b200.headnorm_gate(h, o, w2, eps=1e-6), g[f"hng_{tag}_out"], dt)


@pytest.mark.parametrize("tag,rows,D", [("bf16", 37, 4096), ("bf16", 5, 8192), ("bf16", 64, 512), ("f32", 9, 512),
                                        ("f32", 3, 4096), ("bf16", 1, 8)])
@pytest.mark.parametrize("residual", [False, True])
def test_add_rmsnorm_matches_oracle(tag, rows, D, residual):
    import xlstm_b200
    dt = DT[tag]
    g = torch.Generator().manual_seed(rows * 131 + D)
    x = (3.0 * torch.randn(rows, D, generator=g)).to(dt)
    y = torch.randn(rows, D, generator=g).to(dt) if residual else None
    w = (1.0 + 0.2 * torch.randn(D, generator=g)).to(dt)
    want_x, want_n = O.add_rmsnorm(x, w, y, eps=1e-6)
    got_x, got_n = xlstm_b200.add_rmsnorm(x.cuda(), w.cuda(), None if y is None else y.cuda(), eps=1e-6)
    assert torch.equal(got_x.cpu(), want_x)
    _close(got_n, want_n, dt)


def test_add_rmsnorm_in_place_and_batched_shape():
    import xlstm_b200
    g = torch.Generator().manual_seed(3)
    x = torch.randn(2, 7, 1024, generator=g).bfloat16()
    y = torch.randn(2, 7, 1024, generator=g).bfloat16()
    w = torch.ones(1024).bfloat16()
    want_x, want_n = O.add_rmsnorm(x, w, y)
    xd = x.cuda()
    got_x, got_n = xlstm_b200.add_rmsnorm(xd, w.cuda(), y.cuda(), inplace=True)
    assert got_x.data_ptr() == xd.data_ptr() and got_n.shape == x.shape
    assert torch.equal(xd.cpu(), want_x)
    _close(got_n, want_n, torch.bfloat16)


@pytest.mark.parametrize("tag,B,NH,S,DH", [("bf16", 2, 8, 33, 512), ("bf16", 1, 4, 1, 512), ("f32", 3, 4, 17, 128),
                                           ("bf16", 2, 2, 5, 1024), ("f32", 1, 2, 3, 512), ("bf16", 1, 3, 7, 64)])
def test_headnorm_gate_matches_oracle_on_strided_views(tag, B, NH, S, DH):
    import xlstm_b200
    dt = DT[tag]
    g = torch.Generator().manual_seed(B * 1000 + S * 10 + NH)
    h = (2.0 * torch.randn(B, NH, S, DH, generator=g) + 0.3).to(dt)
    wide = (2.0 * torch.randn(B, S, 3 * NH * DH, generator=g)).to(dt)   # the gate is a column slice of a wider projection
    w = (1.0 + 0.2 * torch.randn(NH * DH, generator=g)).to(dt)
    o = wide[..., 2 * NH * DH:]
    want = O.headnorm_gate(h, o, w, eps=1e-6)
    got = xlstm_b200.headnorm_gate(h.cuda(), wide.cuda()[..., 2 * NH * DH:], w.cuda(), eps=1e-6)
    _close(got, want, dt)
    # the same values through a token-major buffer viewed as (B, NH, S, DH), as the decode step produces them
    hs = h.transpose(1, 2).contiguous().cuda().transpose(1, 2)
    _close(xlstm_b200.headnorm_gate(hs, o.cuda(), w.cuda(), eps=1e-6), want, dt)


def test_unsupported_widths_are_refused_before_launch():
    import xlstm_b200
    from xlstm_b200._lib import XlError
    with pytest.raises(XlError):
        xlstm_b200.add_rmsnorm(torch.zeros(2, 12, device="cuda", dtype=torch.bfloat16), torch.ones(12, device="cuda", dtype=torch.bfloat16))
    with pytest.raises(XlError):
        xlstm_b200.add_rmsnorm(torch.zeros(2, 16384, device="cuda", dtype=torch.bfloat16), torch.ones(16384, device="cuda", dtype=torch.bfloat16))
    with pytest.raises(XlError):
        xlstm_b200.headnorm_gate(torch.zeros(1, 1, 1, 2048, device="cuda", dtype=torch.bfloat16),
                                 torch.zeros(1, 1, 2048, device="cuda", dtype=torch.bfloat16),
                                 torch.ones(2048, device="cuda", dtype=torch.bfloat16))


@pytest.mark.parametrize("tag", ["f32", "bf16"])
def test_soft_cap_matches_oracle_and_reference_fixture(tag):
    import xlstm_b200
    g, dt = load_golden("layer_ops"), DT[tag]
    x = g[f"cap_{tag}_x"].to(dt)
    for cap in (15.0, 30.0):
        got = xlstm_b200.soft_cap(x.cuda(), cap)
        got32 = xlstm_b200.soft_cap(x.cuda(), cap, out_float32=True)
        assert got.dtype == dt and got32.dtype == torch.float32
        assert torch.equal(got32.cpu(), got.float().cpu())
        want = g[f"cap_{tag}_{int(cap)}"]
        diff = (got.float().cpu() - want).abs()
        if tag == "bf16":   # tanhf on the device and on the host may differ in the last fp32 bit before the bf16 rounding
            assert (diff <= want.abs() * 2.0 ** -7).all() and (diff == 0).float().mean().item() > 0.99
        else:
            assert float(diff.max()) <= 1e-5
    if tag == "bf16":   # fp32 arithmetic on bf16 inputs
        got = xlstm_b200.soft_cap(x.cuda(), 15.0, out_float32=True, float32_math=True)
        _close(got, O.soft_cap(x.float(), 15.0), torch.float32)
    big = torch.randn(3, 1000003, generator=torch.Generator().manual_seed(1)) * 40
    _close(xlstm_b200.soft_cap(big.cuda(), 30.0), O.soft_cap(big, 30.0), torch.float32)


@pytest.mark.parametrize("tag", ["f32", "bf16"])
def test_causal_conv1d_kernel_matches_reference_module_fixture(tag):
    import xlstm_b200
    g, dt = load_golden("conv"), DT[tag]
    x, w, b = (g[f"{tag}_{k}"].to(dt).cuda() for k in "xwb")
    _close(xlstm_b200.causal_conv1d(x, w, b), g[f"{tag}_rows"], dt)
    _close(xlstm_b200.causal_conv1d(x, w, b, cu_seqlens=g["cu"].tolist()), g[f"{tag}_packed"], dt)


@pytest.mark.parametrize("tag,B,S,F_,K,bias,silu", [("bf16", 3, 200, 1024, 4, True, True), ("bf16", 2, 70, 72, 3, False, True),
                                                   ("f32", 2, 129, 260, 4, True, False), ("bf16", 1, 1, 8, 8, True, True),
                                                   ("f32", 1, 65, 4, 1, True, True)])
def test_causal_conv1d_kernel_matches_oracle_with_document_boundaries(tag, B, S, F_, K, bias, silu):
    """Boundaries at tile edges, inside tiles, back to back (empty documents) and at row ends; strided input."""
    import xlstm_b200
    dt = DT[tag]
    g = torch.Generator().manual_seed(B * 1000 + S + F_)
    wide = (2.0 * torch.randn(B, S, F_ + 16, generator=g)).to(dt)
    x = wide[:, :, 8:8 + F_] if F_ % 8 == 0 else wide[:, :, :F_].contiguous()   # a column slice of a wider buffer
    w = torch.randn(F_, K, generator=g).to(dt)
    b = (0.3 * torch.randn(F_, generator=g)).to(dt) if bias else None
    cuts = sorted(set([0, B * S] + [r * S for r in range(B)] + [min(B * S, c) for c in (1, 3, 3, 63, 64, 65, 127, 128, 128, S - 1)]))
    cuts = cuts[:1] + [c for c in cuts[1:] for _ in range(2 if c == 64 else 1)]   # an empty document at offset 64
    cuts = sorted(c for c in cuts if c <= B * S)
    for cu in (None, cuts):
        want = O.causal_conv1d(x, w, b, cu_seqlens=cu, silu=silu)
        got = xlstm_b200.causal_conv1d(x.cuda(), w.cuda(), None if b is None else b.cuda(), cu_seqlens=cu, silu=silu)
        _close(got, want, dt)


@pytest.mark.parametrize("tag", ["bf16", "f32"])
@pytest.mark.parametrize("rows,V", [(8, 50304), (1, 50304), (300, 2048), (3, 1000), (5, 7)])
def test_softcap_argmax_kernel_equals_argmax_of_the_capped_logits(tag, rows, V):
    """tokens = argmax(soft_cap(logits, 30)) with the reference's rounding and torch.argmax's tie rule.  The inputs are
    scaled so that many capped values round to the same maximum: the first of them has to win.  Two calls in a row
    share the scratch area (its counters must come back to zero)."""
    import xlstm_b200
    dt = DT[tag]
    g = torch.Generator().manual_seed(rows * 7 + V)
    for scale in (4.0, 40.0):
        x = (scale * torch.randn(rows, V, generator=g)).to(dt)
        want = torch.argmax(O.soft_cap(x, 30.0), dim=-1)
        for _ in range(2):
            got = xlstm_b200.softcap_argmax(x.cuda(), 30.0)
            assert got.dtype == torch.int64 and torch.equal(got.cpu(), want)
    # a strided view (the last position of a (B, S, V) tensor)
    y = (4.0 * torch.randn(4, 3, V, generator=g)).to(dt)
    assert torch.equal(xlstm_b200.softcap_argmax(y.cuda()[:, -1], 30.0).cpu(), torch.argmax(O.soft_cap(y[:, -1], 30.0), dim=-1))


@pytest.mark.parametrize("tag", ["bf16", "f32"])
def test_swiglu_and_strided_biased_soft_cap_match_oracle(tag):
    """The two kernels that take launches out of the decode step: the feed-forward's gating on the stacked
    up-projection, and the soft cap reading the gate columns straight out of the stacked q/k/v/o/gate projection
    (strided rows) with the gate bias added on the way."""
    import xlstm_b200
    dt = DT[tag]
    g = torch.Generator().manual_seed(17)
    for rows, F_ in ((8, 10944), (300, 1368), (1, 8)):
        gz = (2.0 * torch.randn(rows, 2 * F_, generator=g)).to(dt)
        _close(xlstm_b200.swiglu(gz.cuda()), O.swiglu(gz), dt)
    wide = (8.0 * torch.randn(5, 7, 12288 + 16, generator=g)).to(dt)
    bias = torch.randn(16, generator=g).to(dt)
    gates = wide[..., 12288:]
    want = O.soft_cap(gates, 15.0, out_float32=True, bias=bias)
    got = xlstm_b200.soft_cap(wide.cuda()[..., 12288:], 15.0, out_float32=True, bias=bias.cuda())
    assert got.shape == want.shape and got.dtype == torch.float32
    _close(got, want, torch.float32 if tag == "f32" else dt)
    # fp32 arithmetic on the (dtype-rounded) biased input, as the model mirror uses it for the gates
    got2 = xlstm_b200.soft_cap(wide.cuda()[..., 12288:], 15.0, out_float32=True, float32_math=True, bias=bias.cuda())
    pre = (gates.float() + bias.float()).to(dt).float()
    assert float((got2.cpu() - 15.0 * torch.tanh(pre / 15.0)).abs().max()) < 1e-5


@pytest.mark.parametrize("tag", ["bf16", "f32"])
def test_head_group_norm_without_gate_matches_torch_group_norm(tag):
    """The epilogue of the sLSTM layer: per-head group norm of the (B,NH,S,DH) cell output, against torch's own
    ``F.group_norm`` on the transposed copy (what the reference module calls) and against the oracle."""
    import xlstm_b200
    dt = DT[tag]
    g = torch.Generator().manual_seed(23)
    B, NH, S, DH = 3, 4, 37, 256
    h = (2.0 * torch.randn(B, NH, S, DH, generator=g) + 0.3).to(dt)
    w = (1.0 + 0.1 * torch.randn(NH * DH, generator=g)).to(dt)
    got = xlstm_b200.headnorm_gate(h.cuda(), None, w.cuda(), eps=1e-5)
    want = torch.nn.functional.group_norm(h.transpose(1, 2).reshape(B * S, NH * DH).float(), NH, w.float(), None, 1e-5).to(dt)
    _close(got.reshape(B * S, NH * DH), want, dt)
    _close(got, O.head_group_norm(h, w, 1e-5), dt)


@pytest.mark.parametrize("tag", ["a", "b"])
def test_headwise_proj_kernel_matches_reference_modules_fixture(tag):
    """The four gate projections of the reference's sLSTM layer and their concatenation, in one launch."""
    import xlstm_b200
    g = load_golden("headwise")
    bf = lambda t: t.view(torch.bfloat16)
    x, xc, want = bf(g[f"{tag}_x"]).cuda(), bf(g[f"{tag}_xc"]).cuda(), bf(g[f"{tag}_y"])
    got = xlstm_b200.headwise_proj([x, xc], [bf(g[f"{tag}_w{i}"]).cuda() for i in range(4)], [1, 1, 0, 0])
    xlstm_b200.check_device_status()
    assert got.shape == want.shape
    _close(got, want.float(), torch.bfloat16)


@pytest.mark.parametrize("rows,NH,DH,nslots", [(16 * 2048 // 8, 4, 256, 4), (1, 4, 256, 4), (129, 2, 128, 3), (300, 5, 64, 1), (127, 1, 256, 2),
                                                 (300, 2, 128, 4), (641, 1, 256, 4)])
def test_headwise_proj_kernel_matches_oracle(rows, NH, DH, nslots):
    """Row counts around the 128-row tile (pairs of tiles share the weight tiles from 129 rows on: an odd number of tiles
    leaves half a pair empty), all three block sizes, fewer than four slots, a strided second input."""
    import xlstm_b200
    g = torch.Generator().manual_seed(rows + NH + DH)
    D = NH * DH
    x = torch.randn(rows, D, generator=g).bfloat16()
    wide = torch.randn(rows, D + 64, generator=g).bfloat16()
    xc = wide[:, 32:32 + D]                     # a column slice of a wider buffer: row stride D + 64
    ws = [(torch.randn(NH, DH, DH, generator=g) / DH ** 0.5).bfloat16() for _ in range(nslots)]
    sel = [1, 1, 0, 0][:nslots]
    want = O.headwise_proj([x, xc], ws, sel)
    got = xlstm_b200.headwise_proj([x.cuda(), wide.cuda()[:, 32:32 + D]], [w.cuda() for w in ws], sel)
    xlstm_b200.check_device_status()
    # one bf16 ulp, plus an absolute term for sums that cancel (fp32 accumulation in another order)
    diff = (got.float().cpu() - want.float()).abs()
    assert (diff <= want.float().abs() * 2.0 ** -7 + 1e-4).all(), float(diff.max())
    assert rel_l2(got.float().cpu(), want.float()) < 2e-3
    # a (B, S, D) input comes back as (B, S, n * D)
    if rows % 2 == 0:
        got3 = xlstm_b200.headwise_proj([x.cuda().view(2, rows // 2, D)], [ws[0].cuda()])
        assert got3.shape == (2, rows // 2, D)
        assert torch.equal(got3.reshape(rows, D), xlstm_b200.headwise_proj([x.cuda()], [ws[0].cuda()]))
