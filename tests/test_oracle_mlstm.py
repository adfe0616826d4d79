"""The CPU oracle against fixtures produced by the reference's own code
(tests/golden/make_golden.py), plus the self-consistency checks the reference's
tests use (chunkwise == recurrent, tests/template_chunkwise_vs_recurrent.py)."""
import math

import pytest
import torch

from conftest import load_golden, rel_l2
from oracle import mlstm as O

TOL = 2e-5  # fp32 restatement vs fp32 reference, relative L2


def test_chunkwise_zero_state_matches_reference():
    g = load_golden("mlstm_chunk_zero")
    h, (c, n, m) = O.mlstm_chunkwise(g["q"], g["k"], g["v"], g["i"], g["f"])
    assert rel_l2(h, g["h"]) < TOL
    assert rel_l2(c, g["c"]) < TOL
    assert rel_l2(n, g["n"]) < TOL
    assert torch.allclose(m[..., 0], g["m"], atol=1e-5)


def test_chunkwise_initial_state_matches_reference():
    g = load_golden("mlstm_chunk_init")
    h, (c, n, m) = O.mlstm_chunkwise(g["q"], g["k"], g["v"], g["i"], g["f"], g["c0"], g["n0"], g["m0"])
    assert rel_l2(h, g["h"]) < TOL
    assert rel_l2(c, g["c"]) < TOL
    assert rel_l2(n, g["n"]) < TOL
    assert torch.allclose(m[..., 0], g["m"], atol=1e-5)


def test_step_chain_matches_reference():
    g = load_golden("mlstm_step_chain")
    h, (c, n, m) = O.mlstm_sequence(g["q"], g["k"], g["v"], g["i"], g["f"])
    dh = g["q"].shape[-1]
    assert rel_l2(h, g["h"]) < TOL
    # the reference's step function stores keys divided by sqrt(DH) in C and n
    assert rel_l2(c / math.sqrt(dh), g["c_kscaled"]) < TOL
    assert rel_l2(n / math.sqrt(dh), g["n_kscaled"]) < TOL
    assert torch.allclose(m[..., 0], g["m"], atol=1e-5)


def test_third_party_cross_check_rectangular_heads():
    g = load_golden("hf_chunk")
    h, (c, n, m) = O.mlstm_chunkwise(g["q"], g["k"], g["v"], g["i"], g["f"])
    assert rel_l2(h, g["h"]) < TOL and rel_l2(c, g["c"]) < TOL and rel_l2(n, g["n"]) < TOL
    assert torch.allclose(m, g["m"], atol=1e-5)
    g = load_golden("hf_seq")
    h, (c, n, m) = O.mlstm_sequence(g["q"], g["k"], g["v"], g["i"], g["f"], g["c0"], g["n0"], g["m0"])
    assert rel_l2(h, g["h"]) < TOL and rel_l2(c, g["c"]) < TOL and rel_l2(n, g["n"]) < TOL
    assert torch.allclose(m, g["m"], atol=1e-5)


@pytest.mark.parametrize("S,chunk", [(64, 64), (256, 64), (128, 32), (150, 64), (1, 64), (63, 64)])
def test_forms_agree(S, chunk):
    torch.manual_seed(S)
    B, NH, DQ, DV = 2, 3, 16, 24
    q, k = torch.randn(B, NH, S, DQ), torch.randn(B, NH, S, DQ)
    v, i, f = torch.randn(B, NH, S, DV), torch.randn(B, NH, S), torch.randn(B, NH, S) + 2
    h_seq, st_seq = O.mlstm_sequence(q, k, v, i, f)
    h_inf, st_inf = O.mlstm_inference(q, k, v, i, f, chunk_size=chunk)
    assert rel_l2(h_inf, h_seq) < 1e-4
    for a, b in zip(st_inf, st_seq):
        assert rel_l2(a, b) < 1e-4
    assert rel_l2(O.mlstm_parallel(q, k, v, i, f), h_seq) < 1e-4


def test_packed_equals_per_document_and_resets_state():
    torch.manual_seed(0)
    NH, DQ, DV = 2, 16, 16
    cu = [0, 5, 5, 70, 200, 264]
    T = cu[-1]
    q, k, v = torch.randn(NH, T, DQ), torch.randn(NH, T, DQ), torch.randn(NH, T, DV)
    i, f = torch.randn(NH, T), torch.randn(NH, T) + 1
    h, (c, n, m) = O.mlstm_packed(q, k, v, i, f, cu)
    assert h.shape == (NH, T, DV) and c.shape == (5, NH, DQ, DV)
    # an empty document leaves the zero state
    assert float(c[1].abs().max()) == 0.0 and float(m[1].abs().max()) == 0.0
    # document 3 alone
    s, e = cu[3], cu[4]
    h3, st3 = O.mlstm_sequence(q[None, :, s:e], k[None, :, s:e], v[None, :, s:e], i[None, :, s:e], f[None, :, s:e])
    assert rel_l2(h[:, s:e], h3[0]) < 1e-4 and rel_l2(c[3], st3[0][0]) < 1e-4
