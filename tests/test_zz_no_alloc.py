"""pj_index_records_static: the record index for callers that cannot allocate device memory.

Some hosts of this library run where cudaMalloc / cudaFree are off limits: the device memory belongs to an
embedding runtime's pool, the process froze its allocations after start-up, or the calling thread cannot
afford the implicit synchronisation of an allocation. For them the library keeps the index scratch in a
fixed array inside its own image. This test drives that entry point through the C ABI with device buffers
only and checks it against the ordinary pj_index_records, twice in a row on inputs of different sizes so
that whatever the first call left in the shared array cannot leak into the second.

Collected last on purpose (file name), so a run that stops at the first failure has already run the rest.
"""
import ctypes as C

import numpy as np
import pytest

from pj_testlib import abi, pj

pytestmark = pytest.mark.gpu


def reference_index(ctx, d_text, cap):
    import torch

    d_rs = torch.zeros(cap, dtype=torch.int64, device=d_text.device)
    n = ctx.index_records(d_text, d_rs, allow_capacity=True)
    return n, d_rs.cpu().numpy().view(np.uint64)


def test_static_index_matches_the_allocating_one_twice_in_a_row(ctx, oracle):
    import torch

    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    inputs = [pj.gen_text(abi.PJ_SCHEMA_MIXED, 71, 0, 40000, abi.PJ_GEN_WHITESPACE | abi.PJ_GEN_MALFORMED),   # ~10 MB
              np.concatenate([np.frombuffer(b"\n \r\n{}\n\n", np.uint8), pj.gen_text(abi.PJ_SCHEMA_PET, 72, 0, 900, 0)])]  # smaller, blank lines
    for text in inputs:
        d_text = torch.from_numpy(np.ascontiguousarray(text)).cuda()
        cap = int(np.count_nonzero(text == 10)) + 8
        want_n, want = reference_index(ctx, d_text, cap)
        checker = oracle.index(np.ascontiguousarray(text))  # ... and both against the CPU checker's line index
        assert want_n == checker.size and np.array_equal(want[:want_n], checker)
        d_rs = torch.full((cap,), -1, dtype=torch.int64, device="cuda")
        d_n = torch.full((1,), -1, dtype=torch.int64, device="cuda")
        pj.index_records_static(d_text, d_rs, d_n, stream)
        torch.cuda.synchronize()
        assert int(d_n.item()) == want_n > 0
        assert np.array_equal(d_rs.cpu().numpy().view(np.uint64)[:want_n], want[:want_n])
        # a buffer that is too small: the true count is still reported, only `cap` offsets are stored
        d_small = torch.full((10,), -1, dtype=torch.int64, device="cuda")
        pj.index_records_static(d_text, d_small, d_n, stream)
        torch.cuda.synchronize()
        assert int(d_n.item()) == want_n and np.array_equal(d_small.cpu().numpy().view(np.uint64), want[:10])


def test_static_index_rejects_what_its_fixed_scratch_cannot_serve(native):
    L = native.lib()
    too_big = (1 << 30) + 1
    n = C.c_uint64()
    # size is checked before anything touches the device: no GPU memory is needed for this call
    st = L.pj_index_records_static(C.c_void_p(16), too_big, C.c_void_p(16), 1, C.byref(n), None)
    assert st == abi.PJ_ERR_TOO_LARGE
    assert b"fixed scratch" in L.pj_last_error(None)
    assert L.pj_index_records_static(None, 5, None, 0, C.byref(n), None) == abi.PJ_ERR_ARG
