"""Parity of the CUDA mLSTM kernels (through the C ABI) with the CPU oracle on identical seeded inputs.

Tolerances (relative L2): bf16 outputs and states <= 1e-2, fp32 mode <= 1e-4.
The bf16 oracle is "inputs rounded to bf16, arithmetic in fp32".
"""
import math

import pytest
import torch

from conftest import load_golden, rel_l2
from oracle import mlstm as O

pytestmark = pytest.mark.gpu
TOL_BF16, TOL_F32 = 1e-2, 1e-4


def _inputs(seed, B, NH, S, DQ, DV, dtype, f_mean=3.0):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, NH, S, DQ, generator=g) / math.sqrt(DQ) * math.sqrt(DQ) ** 0  # N(0,1); scale applied below
    k = torch.randn(B, NH, S, DQ, generator=g)
    v = torch.randn(B, NH, S, DV, generator=g)
    i = torch.randn(B, NH, S, generator=g)
    f = torch.randn(B, NH, S, generator=g) + f_mean
    q, k, v = (t.to(dtype) for t in (q, k, v))
    return q, k, v, i, f


def _state(seed, N, NH, DQ, DV):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(N, NH, DQ, DV, generator=g), torch.randn(N, NH, DQ, generator=g), torch.randn(N, NH, 1, generator=g))


def _cuda(*ts):
    return [None if t is None else t.cuda() for t in ts]


def _check(h, st, h_ref, st_ref, tol):
    assert torch.isfinite(h.float()).all()
    assert rel_l2(h.float().cpu(), h_ref) < tol, rel_l2(h.float().cpu(), h_ref)
    for a, b, name in zip(st, st_ref, "cnm"):
        a = a.float().cpu().reshape(b.shape)
        if name == "m":
            assert torch.allclose(a, b, atol=1e-3, rtol=1e-4), (a - b).abs().max()
        else:
            assert rel_l2(a, b) < tol, (name, rel_l2(a, b))


# ------------------------------------------------------------------------------------------------ step
@pytest.mark.parametrize("dtype,tol", [(torch.float32, TOL_F32), (torch.bfloat16, TOL_BF16)])
@pytest.mark.parametrize("B,NH,DQ,DV", [(3, 2, 64, 128), (2, 8, 256, 512), (1, 1, 32, 36)])
def test_step_matches_oracle(dtype, tol, B, NH, DQ, DV):
    import xlstm_b200
    q, k, v, i, f = _inputs(1, B, NH, 1, DQ, DV, dtype, f_mean=1.0)
    c0, n0, m0 = _state(2, B, NH, DQ, DV)
    h_ref, st_ref = O.mlstm_step(q[:, :, 0], k[:, :, 0], v[:, :, 0], i, f, c0, n0, m0)
    qc, kc, vc, ic, fc, cc, nc, mc = _cuda(q[:, :, 0], k[:, :, 0], v[:, :, 0], i, f, c0.clone(), n0, m0)
    h, st = xlstm_b200.mlstm_step(qc, kc, vc, ic, fc, cc, nc, mc)
    assert st[0] is cc  # the large state is updated in place and handed back as the same object
    _check(h, st, h_ref, st_ref, tol)
    # from the zero state
    h_ref, st_ref = O.mlstm_step(q[:, :, 0], k[:, :, 0], v[:, :, 0], i, f)
    h, st = xlstm_b200.mlstm_step(qc, kc, vc, ic, fc, None, None, None)
    _check(h, st, h_ref, st_ref, tol)


def test_step_slots_and_strided_views():
    import xlstm_b200
    B, NH, DQ, DV, N = 3, 2, 64, 128, 5
    q, k, v, i, f = _inputs(3, B, NH, 1, DQ, DV, torch.bfloat16)
    c0, n0, m0 = _state(4, N, NH, DQ, DV)
    slot = torch.tensor([4, 0, 2], dtype=torch.int32)
    h_ref, st_ref = O.mlstm_step(q[:, :, 0], k[:, :, 0], v[:, :, 0], i, f, c0[slot.long()], n0[slot.long()], m0[slot.long()])
    # q,k,v as slices of one fused projection buffer (B, NH*(2DQ+DV)) -> strided (B,NH,D) views
    fused = torch.cat([q[:, :, 0].reshape(B, -1), k[:, :, 0].reshape(B, -1), v[:, :, 0].reshape(B, -1)], dim=1).cuda()
    qv = fused[:, : NH * DQ].view(B, NH, DQ)
    kv = fused[:, NH * DQ: 2 * NH * DQ].view(B, NH, DQ)
    vv = fused[:, 2 * NH * DQ:].view(B, NH, DV)
    cc, nc, mc = c0.cuda(), n0.cuda(), m0.cuda()
    h, (c, n, m) = xlstm_b200.mlstm_step(qv, kv, vv, i.cuda(), f.cuda(), cc, nc, mc, slot=slot.cuda())
    _check(h, (c[slot.long().cuda()], n[slot.long().cuda()], m[slot.long().cuda()]), h_ref, st_ref, TOL_BF16)
    untouched = torch.tensor([1, 3])
    assert torch.equal(c[untouched.cuda()].cpu(), c0[untouched]) and torch.equal(n[untouched.cuda()].cpu(), n0[untouched])


# ------------------------------------------------------------------------------------------------ recurrent
@pytest.mark.parametrize("name", ["mlstm_chunk_zero", "mlstm_chunk_init", "hf_chunk", "hf_seq"])
def test_recurrent_fp32_matches_reference_fixtures(name):
    import xlstm_b200
    g = load_golden(name)
    init = _cuda(g.get("c0"), g.get("n0"), g.get("m0"))
    h, st = xlstm_b200.mlstm_sequence(*_cuda(g["q"], g["k"], g["v"], g["i"], g["f"]), *init, kernel="recurrent")
    _check(h, st, g["h"], (g["c"], g["n"], g["m"].reshape(g["c"].shape[0], -1, 1)), TOL_F32)


def test_recurrent_fp32_config1_shape():
    """B=3, NH=4, S=256, DHQK=64, DHV=128, fp32: the cell shape of the small reference model (embedding 512, 4 heads)."""
    import xlstm_b200
    q, k, v, i, f = _inputs(5, 3, 4, 256, 64, 128, torch.float32)
    h_ref, st_ref = O.mlstm_chunkwise(q, k, v, i, f)
    h, st = xlstm_b200.mlstm_sequence(*_cuda(q, k, v, i, f), kernel="auto")  # fp32 -> recurrence
    _check(h, st, h_ref, st_ref, TOL_F32)


# ------------------------------------------------------------------------------------------------ chunkwise (tcgen05)
@pytest.mark.parametrize("B,NH,S,DQ,DV,with_state", [
    (2, 2, 256, 64, 128, False),
    (1, 2, 150, 128, 256, True),     # 2 full chunks + 22-token tail, initial state
    (1, 1, 64, 256, 512, False),
    (2, 3, 1000, 256, 512, True),
    (1, 2, 7, 64, 128, False),       # shorter than one chunk
    (1, 2, 200, 256, 256, True),     # more feature blocks than value slices: no cluster split of the normaliser
    (1, 1, 130, 128, 512, False),    # fewer feature blocks than value slices: likewise
])
def test_chunkwise_matches_oracle(B, NH, S, DQ, DV, with_state):
    import xlstm_b200
    q, k, v, i, f = _inputs(7, B, NH, S, DQ, DV, torch.bfloat16)
    init = _state(8, B, NH, DQ, DV) if with_state else (None, None, None)
    h_ref, st_ref = O.mlstm_inference(q, k, v, i, f, *init)
    h, st = xlstm_b200.mlstm_sequence(*_cuda(q, k, v, i, f), *_cuda(*init), kernel="chunkwise")
    xlstm_b200.check_device_status()
    _check(h, st, h_ref, st_ref, TOL_BF16)


@pytest.mark.parametrize("cluster,DQ,DV", [(4, 256, 512), (2, 128, 256), (2, 256, 512)])
def test_chunkwise_cluster_shared_normaliser_opt_in(cluster, DQ, DV):
    """XL_CW_CLUSTER=2|4 lets the value slices of a head share the normaliser work through a thread-block cluster
    (read once per process, hence the child process).  Same results as the default path."""
    import os, subprocess, sys
    code = (
        "import sys, torch; sys.path.insert(0, %r); sys.path.insert(0, %r)\n"
        "import xlstm_b200\n"
        "from oracle import mlstm as O\n"
        "from conftest import rel_l2\n"
        "from test_gpu_mlstm import _inputs, _state\n"
        "q, k, v, i, f = _inputs(31, 2, 2, 300, %d, %d, torch.bfloat16)\n"
        "init = _state(32, 2, 2, %d, %d)\n"
        "h_ref, st_ref = O.mlstm_inference(q, k, v, i, f, *init)\n"
        "h, st = xlstm_b200.mlstm_sequence(*[t.cuda() for t in (q, k, v, i, f)], *[t.cuda() for t in init], kernel='chunkwise')\n"
        "xlstm_b200.check_device_status()\n"
        "errs = [rel_l2(h.float().cpu(), h_ref.float())] + [rel_l2(a.cpu(), b) for a, b in zip(st, st_ref)]\n"
        "print('ERRS', errs)\n"
        "assert max(errs) < 1e-2, errs\n"
    ) % (os.path.dirname(os.path.dirname(os.path.abspath(__file__))), os.path.dirname(os.path.abspath(__file__)), DQ, DV, DQ, DV)
    env = dict(os.environ, XL_CW_CLUSTER=str(cluster))
    res = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]


def test_chunkwise_harsh_gates_stay_finite_and_match():
    """Forget gates around -6 (strong decay) and input gates with a wide spread exercise the stabilisers."""
    import xlstm_b200
    B, NH, S, DQ, DV = 1, 2, 320, 64, 128
    q, k, v, i, f = _inputs(9, B, NH, S, DQ, DV, torch.bfloat16, f_mean=-6.0)
    i = i * 6.0
    h_ref, st_ref = O.mlstm_inference(q, k, v, i, f)
    h, st = xlstm_b200.mlstm_sequence(*_cuda(q, k, v, i, f), kernel="chunkwise")
    _check(h, st, h_ref, st_ref, TOL_BF16)


@pytest.mark.parametrize("DQ,DV", [(64, 128), (256, 512)])
@pytest.mark.parametrize("jump", [20.0, 40.0, 120.0])
def test_chunkwise_stabiliser_jumps_inside_a_chunk(jump, DQ, DV):
    """An input gate that leaps by `jump` nats in the middle of a chunk: the rows before the leap must keep their
    own scale (the kernel switches that chunk to its per-row frame), the rows after it forget the past."""
    import xlstm_b200
    B, NH, S = 1, 2, 256
    q, k, v, i, f = _inputs(21, B, NH, S, DQ, DV, torch.bfloat16)
    # a common component in q and k keeps q.n away from zero, so that h is well conditioned where only a few
    # tokens carry weight
    q = (q.float() + 1.0).to(torch.bfloat16)
    k = (k.float() + 1.0).to(torch.bfloat16)
    i = i.clone()
    i[:, :, 100:] += jump          # inside chunk 1
    i[:, 1, 200:] -= 2 * jump      # and back down inside chunk 3 for one head
    h_ref, st_ref = O.mlstm_inference(q, k, v, i, f)
    h, st = xlstm_b200.mlstm_sequence(*_cuda(q, k, v, i, f), kernel="chunkwise")
    assert torch.isfinite(h.float()).all()
    _check(h, st, h_ref, st_ref, TOL_BF16)
    # the rows before the leap alone
    assert rel_l2(h[:, :, 64:100].float().cpu(), h_ref[:, :, 64:100].float()) <= TOL_BF16


def test_chunkwise_transposed_views_like_the_reference_layer():
    """q,k,v arrive as (B,S,NH*D) projections viewed as (B,NH,S,D) -- xlstm_large/model.py:415-419."""
    import xlstm_b200
    B, NH, S, DQ, DV = 2, 4, 192, 64, 128
    q, k, v, i, f = _inputs(10, B, NH, S, DQ, DV, torch.bfloat16)
    h_ref, st_ref = O.mlstm_inference(q, k, v, i, f)
    qc = q.transpose(1, 2).reshape(B, S, NH * DQ).cuda().reshape(B, S, NH, DQ).transpose(1, 2)
    kc = k.transpose(1, 2).reshape(B, S, NH * DQ).cuda().reshape(B, S, NH, DQ).transpose(1, 2)
    vc = v.transpose(1, 2).reshape(B, S, NH * DV).cuda().reshape(B, S, NH, DV).transpose(1, 2)
    ic = i.transpose(1, 2).contiguous().cuda().transpose(1, 2)
    fc = f.transpose(1, 2).contiguous().cuda().transpose(1, 2)
    assert not qc.is_contiguous()
    h, st = xlstm_b200.mlstm_sequence(qc, kc, vc, ic, fc, kernel="chunkwise")
    _check(h, st, h_ref, st_ref, TOL_BF16)


@pytest.mark.parametrize("kernel,dtype,tol", [("chunkwise", torch.bfloat16, TOL_BF16), ("recurrent", torch.float32, TOL_F32)])
def test_packed_documents_reset_state_in_kernel(kernel, dtype, tol):
    """Ragged documents packed into rows, boundaries anywhere (also inside a 64-token chunk), an empty
    document, and a document that ends exactly at a row end.  Oracle = each document alone."""
    import xlstm_b200
    B, NH, S, DQ, DV = 2, 2, 256, 64, 128
    cu = [0, 5, 5, 70, 200, 256, 256 + 64, 256 + 191, 512]
    q, k, v, i, f = _inputs(11, B, NH, S, DQ, DV, dtype)
    flat = lambda t: t.transpose(0, 1).reshape(NH, B * S, *t.shape[3:])
    h_ref, st_ref = O.mlstm_packed(flat(q), flat(k), flat(v), flat(i), flat(f), cu)
    h, st = xlstm_b200.mlstm_sequence(*_cuda(q, k, v, i, f), cu_seqlens=cu, kernel=kernel)
    xlstm_b200.check_device_status()
    assert st[0].shape == (len(cu) - 1, NH, DQ, DV)
    _check(flat(h.cpu()), st, h_ref, st_ref, tol)


def test_chunkwise_full_size_config2_properties():
    """The benchmark shape at full size (B=4, NH=8, S=8192, DHQK=256, DHV=512, bf16: xLSTM-7B heads).  Checks:
    (1) the tensor-core kernel agrees with the on-device fp32 recurrence for one (batch, head) pair,
    (2) splitting the sequence in two calls that hand the state over gives the same result,
    (3) batch rows / heads are independent (same inputs in two rows -> identical outputs),
    (4) two full rows against the CPU oracle (h, C, n, m)."""
    import xlstm_b200
    B, NH, S, DQ, DV = 4, 8, 8192, 256, 512
    g = torch.Generator(device="cuda").manual_seed(0)
    q = (torch.randn(B, NH, S, DQ, generator=g, device="cuda") / math.sqrt(DQ)).bfloat16()
    k = (torch.randn(B, NH, S, DQ, generator=g, device="cuda") / math.sqrt(DQ)).bfloat16()
    v = torch.randn(B, NH, S, DV, generator=g, device="cuda").bfloat16()
    i = torch.randn(B, NH, S, generator=g, device="cuda")
    f = torch.randn(B, NH, S, generator=g, device="cuda") + 3.0
    q[3], k[3], v[3], i[3], f[3] = q[0], k[0], v[0], i[0], f[0]
    h, (c, n, m) = xlstm_b200.mlstm_sequence(q, k, v, i, f, kernel="chunkwise")
    xlstm_b200.check_device_status()
    assert torch.isfinite(h.float()).all() and torch.isfinite(c).all()
    assert torch.equal(h[3], h[0]) and torch.equal(c[3], c[0])
    sl = (slice(1, 2), slice(2, 3))
    hr, (cr, nr, mr) = xlstm_b200.mlstm_sequence(q[sl], k[sl], v[sl], i[sl], f[sl], kernel="recurrent")
    assert rel_l2(h[sl].float(), hr.float()) < TOL_BF16
    assert rel_l2(c[sl], cr) < TOL_BF16 and rel_l2(n[sl], nr) < TOL_BF16
    assert torch.allclose(m[sl], mr, atol=1e-3)
    half = 4096 + 37
    h1, st1 = xlstm_b200.mlstm_sequence(q[:1, :, :half], k[:1, :, :half], v[:1, :, :half], i[:1, :, :half], f[:1, :, :half], kernel="chunkwise")
    h2, st2 = xlstm_b200.mlstm_sequence(q[:1, :, half:], k[:1, :, half:], v[:1, :, half:], i[:1, :, half:], f[:1, :, half:], *st1, kernel="chunkwise")
    assert rel_l2(torch.cat([h1, h2], 2).float(), h[:1].float()) < TOL_BF16
    assert rel_l2(st2[0], c[:1]) < TOL_BF16
    # (4) against the CPU oracle directly: two full rows (all 8 heads, all 8192 tokens) of h and of the final C, n, m
    for row in (1, 2):
        h_ref, (c_ref, n_ref, m_ref) = O.mlstm_inference(q[row:row + 1].cpu(), k[row:row + 1].cpu(), v[row:row + 1].cpu(),
                                                         i[row:row + 1].cpu(), f[row:row + 1].cpu())
        _check(h[row:row + 1], (c[row:row + 1], n[row:row + 1], m[row:row + 1]), h_ref, (c_ref, n_ref, m_ref), TOL_BF16)
        # no drift along the sequence: the last 512 tokens are as close as the whole row
        assert rel_l2(h[row, :, -512:].float().cpu(), h_ref[0, :, -512:]) < TOL_BF16


def test_prefill_from_pinned_host_buffers_equals_device_call():
    """The host-buffer entry (pieces over three streams, uploads / kernels / downloads overlapped) returns what the
    device-resident call returns."""
    import xlstm_b200
    B, NH, S, DQ, DV = 3, 4, 200, 64, 128
    q, k, v, i, f = _inputs(41, B, NH, S, DQ, DV, torch.bfloat16)
    host = [t.pin_memory() for t in (q, k, v, i, f)]
    h_host = torch.empty(B, NH, S, DV, dtype=torch.bfloat16).pin_memory()
    c_host = torch.empty(B, NH, DQ, DV).pin_memory()
    n_host = torch.empty(B, NH, DQ).pin_memory()
    m_host = torch.empty(B, NH, 1).pin_memory()
    xlstm_b200.mlstm_sequence_from_host(*host, h_host, c_host, n_host, m_host)
    torch.cuda.synchronize()
    h, (c, n, m) = xlstm_b200.mlstm_sequence(*_cuda(q, k, v, i, f), kernel="chunkwise")
    assert torch.equal(h_host, h.cpu()) and torch.equal(c_host, c.cpu())
    assert torch.equal(n_host, n.cpu()) and torch.equal(m_host, m.cpu())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("B,NH,DQ,DV,with_slots", [(8, 8, 256, 512, False), (5, 3, 64, 128, True), (2, 2, 128, 1024, True), (3, 4, 32, 40, False)])
def test_fused_decode_cell_equals_cap_step_norm_gate(dtype, B, NH, DQ, DV, with_slots):
    """One kernel for gate soft cap + cell step + per-head norm + output gate against the three separate kernels: the
    states bit for bit (same arithmetic), the gated output up to the summation order of the norm's two sums (the thread
    blocks of a head exchange partial sums through distributed shared memory)."""
    import xlstm_b200
    from xlstm_b200 import ops
    if dtype == torch.float32 and DV > 512:
        pytest.skip("the separate norm kernel takes at most 512 fp32 columns per head")
    g = torch.Generator().manual_seed(B * 100 + NH * 10 + DV)
    rnd = lambda *shape: torch.randn(*shape, generator=g)
    q, k, v = rnd(B, NH, DQ).to(dtype).cuda(), rnd(B, NH, DQ).to(dtype).cuda(), rnd(B, NH, DV).to(dtype).cuda()
    wide = (4.0 * rnd(B, 2 * NH + 24)).to(dtype).cuda()
    gates_raw = wide[:, 8:8 + 2 * NH]                      # a column slice of a wider projection output
    bias = torch.cat([torch.zeros(NH), 3.0 + torch.zeros(NH)]).to(dtype).cuda()
    ogate, w = rnd(B, NH * DV).to(dtype).cuda(), (1.0 + 0.1 * rnd(NH * DV)).to(dtype).cuda()
    N = B + 3 if with_slots else B
    pool = [rnd(N, NH, DQ, DV).cuda(), rnd(N, NH, DQ).cuda(), rnd(N, NH, 1).cuda()]
    slot = None
    if with_slots:
        slot = torch.tensor([N - 1 - 2 * j if j % 3 != 1 else -1 for j in range(B)], dtype=torch.int32)   # every third stream inactive
    # the three kernels
    gates = ops.soft_cap(gates_raw, 15.0, out_float32=True, float32_math=True, bias=bias)
    c1 = [t.clone() for t in pool]
    h, st1 = xlstm_b200.mlstm_step(q, k, v, gates[:, :NH], gates[:, NH:], *c1, slot=slot)
    want = xlstm_b200.headnorm_gate(h[:, :, None], ogate[:, None], w)[:, 0]
    # the one kernel
    c2 = [t.clone() for t in pool]
    got, st2 = ops.mlstm_decode_cell(q, k, v, gates_raw, bias, 15.0, ogate, w, *c2, slot=slot)
    xlstm_b200.check_device_status()
    for a, b_ in zip(st1, st2):
        assert torch.equal(a, b_)
    assert got.shape == (B, NH * DV)
    d = (got.float() - want.float()).abs()
    tol = 2.0 ** -7 if dtype == torch.bfloat16 else 1e-5
    assert (d <= want.float().abs() * tol + 1e-5).all(), float(d.max())
    if with_slots:   # inactive streams: zero output, pool untouched
        idle = [j for j in range(B) if int(slot[j]) < 0]
        assert float(got[idle].float().abs().max()) == 0.0
