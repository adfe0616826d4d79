"""The allocation-free greedy head, through the C ABI, against the entry point that takes caller scratch.

``xl_softcap_argmax_noalloc`` is for callers that have no device memory to lend and may not allocate any: a serving loop
whose buffers were all placed at start-up, a plugin in a host that owns the GPU's memory.  Its scratch is an array built
into the library, shared by every call on the device and keeping whatever the last call left in it; so the check is made
on TWO calls in a row (different inputs, the second with fewer rows, so that it meets the first call's leftovers), and
the tokens must equal those of ``xl_softcap_argmax`` exactly (they are integers).  This file is collected last on
purpose: a run that stops at the first failure has then already run every other test.  It does not depend on them: the
library is loaded here if nobody loaded it before.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(fn, logits, tokens, scratch=None):
    from xlstm_b200 import _lib
    p = _lib.GreedyParams()
    p.logits, p.tokens = logits.data_ptr(), tokens.data_ptr()
    if scratch is not None:
        p.scratch, p.scratch_bytes = scratch.data_ptr(), scratch.numel()
    p.rows, p.V, p.row_stride, p.cap, p.dtype = logits.shape[0], logits.shape[1], logits.stride(0), 30.0, _lib.XL_BF16
    return fn(C.byref(p), torch.cuda.current_stream().cuda_stream)


def test_allocation_free_greedy_head_equals_the_scratch_taking_one_twice_in_a_row():
    from xlstm_b200 import _lib
    lib = _lib.lib()
    torch.cuda.set_device(0)
    assert lib.xl_softcap_argmax_noalloc_max_rows() == 1024
    g = torch.Generator().manual_seed(123)
    for rows, V, scale in ((37, 50304, 6.0), (8, 50304, 40.0)):   # the second call: fewer rows, many ties at the cap
        logits = (scale * torch.randn(rows, V, generator=g)).bfloat16().cuda()
        want = torch.full((rows,), -1, dtype=torch.int64, device="cuda")
        got = torch.full((rows,), -2, dtype=torch.int64, device="cuda")
        scratch = torch.zeros(int(lib.xl_softcap_argmax_scratch_bytes(rows)), dtype=torch.uint8, device="cuda")
        assert _call(lib.xl_softcap_argmax, logits, want, scratch) == 0
        assert _call(lib.xl_softcap_argmax_noalloc, logits, got) == 0
        torch.cuda.synchronize()
        assert torch.equal(got, want)
        assert int(want.min()) >= 0 and int(want.max()) < V
    # beyond the built-in capacity: refused before anything is launched, with a status that says why
    big = torch.zeros(1025, 8, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(1025, dtype=torch.int64, device="cuda")
    rc = _call(lib.xl_softcap_argmax_noalloc, big, out)
    assert rc == -8 and b"capacity" in lib.xl_strerror(rc)
