"""The allocation-free nearest-centroid entry point, called through the C ABI.

Some callers cannot let the library allocate: a loop that files new rows into IVF lists while other
streams are serving queries (cudaMalloc/cudaFree stall the whole device), or a process that has already
given every byte of the GPU to its own buffers.  For them ``vsk_assign_static_dev`` keeps its scratch in a
fixed array inside the library.  It must return exactly what ``vsk_assign_dev`` returns — also on a second
call, when the shared array still holds the first call's keys.

Collected last on purpose (file name), so that a run stopping at the first failure has already run every
other test; it also passes when run alone in a fresh process.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _call(lib, fn, ctx, x, c):
    import torch
    n, d = x.shape
    asg = torch.empty(n, dtype=torch.int32, device=x.device)
    dist = torch.empty(n, dtype=torch.float32, device=x.device)
    torch.cuda.synchronize()   # the library's stream does not wait for torch's: inputs must be complete
    st = fn(ctx, C.c_void_p(x.data_ptr()), n, d, C.c_void_p(c.data_ptr()), c.shape[0],
            C.c_void_p(asg.data_ptr()), C.c_void_p(dist.data_ptr()))
    return st, asg.cpu().numpy(), dist.cpu().numpy()


def test_static_scratch_assign_matches_allocating_entry_point_twice():
    import torch
    from vectorstorekit_b200 import _lib
    lib = _lib.load()
    ctx = C.c_void_p()
    assert lib.vsk_open(0, C.byref(ctx)) == 0
    try:
        g = torch.Generator(device="cuda").manual_seed(99)
        # second call: fewer rows, other centroids — stale keys of the first call lie beyond and beneath it
        for n, d, k in [(70_000, 64, 257), (33_333, 64, 19)]:
            x = torch.randn((n, d), generator=g, device="cuda")
            c = torch.randn((k, d), generator=g, device="cuda")
            st0, a0, d0 = _call(lib, lib.vsk_assign_dev, ctx, x, c)
            st1, a1, d1 = _call(lib, lib.vsk_assign_static_dev, ctx, x, c)
            assert st0 == 0 and st1 == 0, lib.vsk_last_error(ctx)
            # the tolerances of the other assignment tests: the two entry points may sum a row's squares in a
            # different order, which can flip a row that is equally near two centroids to within rounding
            assert np.mean(a1 == a0) > 0.999
            assert np.allclose(d1, d0, rtol=1e-4, atol=1e-4)
            assert a1.min() >= 0 and a1.max() < k
        # the property the entry point exists for: after its first call on the device it allocates nothing.  Free
        # device memory (cudaMemGetInfo) must not move across further calls - also right after the allocating entry
        # point grew its own scratch for a larger batch.
        x = torch.randn((200_000, 64), generator=g, device="cuda")
        c = torch.randn((300, 64), generator=g, device="cuda")
        xs = x[:50_000].contiguous()
        st, _, _ = _call(lib, lib.vsk_assign_dev, ctx, x, c)
        assert st == 0
        outs = [torch.empty(50_000, dtype=torch.int32, device="cuda"), torch.empty(50_000, dtype=torch.float32, device="cuda")]
        torch.cuda.synchronize()
        free0 = torch.cuda.mem_get_info()[0]
        for _ in range(3):
            st = lib.vsk_assign_static_dev(ctx, C.c_void_p(xs.data_ptr()), 50_000, 64, C.c_void_p(c.data_ptr()), 300,
                                           C.c_void_p(outs[0].data_ptr()), C.c_void_p(outs[1].data_ptr()))
            assert st == 0
            assert torch.cuda.mem_get_info()[0] == free0
        # beyond the fixed capacity: refused with a clear message, nothing launched
        big = (1 << 20) + 1
        x = torch.zeros((big, 4), device="cuda")
        c = torch.zeros((2, 4), device="cuda")
        st, _, _ = _call(lib, lib.vsk_assign_static_dev, ctx, x, c)
        assert st == 4  # VSK_ERR_INVALID_BUFFER_SIZE
        assert b"at most 1048576 rows" in lib.vsk_last_error(ctx)
    finally:
        lib.vsk_close(ctx)
