"""Allocation-free dispatch entry point (collected last on purpose).

`asca_moe_dispatch_noalloc` serves callers that may not allocate device memory while they
run (a serving loop that owns all of HBM through its own arena, hosts that forbid cudaMalloc
and cudaFree once requests are flowing because both synchronise the GPU). Its scratch is a fixed array in
the library's device image, shared by every call on that GPU. The test calls it through the C
ABI twice in a row -- the second call sees whatever the first left in the scratch -- and
demands the same integers as the allocating entry point, then checks that an over-size
request is refused with a message instead of overrunning the array.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _dispatch(gpu, fn, ids, e):
    import torch

    t_ids = torch.from_numpy(ids.view(np.int32)).cuda()
    n = ids.size
    perm = torch.full((max(n, 1),), -7, dtype=torch.int32, device="cuda")
    off = torch.full((e + 1,), -7, dtype=torch.int32, device="cuda")
    route = torch.full((max(n, 1),), -7, dtype=torch.int32, device="cuda")
    gpu._call(fn, gpu._ctx, C.c_void_p(t_ids.data_ptr()), C.c_int64(n), C.c_int64(e), C.c_void_p(perm.data_ptr()),
              C.c_void_p(off.data_ptr()), C.c_void_p(route.data_ptr()))
    gpu.sync()
    return perm[:n].cpu().numpy(), off.cpu().numpy(), route[:n].cpu().numpy()


def test_noalloc_dispatch_matches_allocating_entry_point_twice_in_a_row(gpu, orc):
    rs = np.random.RandomState(123)
    # two different problems back to back; the second is smaller, so stale entries of the first
    # stay in the shared scratch beyond what the second call uses
    for n, e, vocab in ((200_000, 64, 256), (5_003, 16, 50_000)):
        ids = rs.randint(0, vocab, size=n).astype(np.uint32)
        want = _dispatch(gpu, "asca_moe_dispatch", ids, e)
        got = _dispatch(gpu, "asca_moe_dispatch_noalloc", ids, e)
        for a, b in zip(got, want):
            assert np.array_equal(a, b)
        assert sorted(got[0].tolist()) == list(range(n))  # a permutation of all tokens
        for a, b in zip(got, orc.moe_dispatch(ids, e)):   # and the CPU oracle's buckets, directly
            assert np.array_equal(a, b)


def test_noalloc_dispatch_rejects_sizes_beyond_its_fixed_scratch(gpu):
    import asca_b200
    import torch

    n, e = 2_000_000, 64  # 1956 segments * 64 experts > 65536 ints
    ids = torch.zeros(n, dtype=torch.int32, device="cuda")
    perm = torch.empty(n, dtype=torch.int32, device="cuda")
    off = torch.empty(e + 1, dtype=torch.int32, device="cuda")
    before = gpu.launch_count()
    with pytest.raises(asca_b200.AscaError) as err:
        gpu._call("asca_moe_dispatch_noalloc", gpu._ctx, C.c_void_p(ids.data_ptr()), C.c_int64(n), C.c_int64(e),
                  C.c_void_p(perm.data_ptr()), C.c_void_p(off.data_ptr()), C.c_void_p(0))
    assert err.value.code == -1 and "must not exceed" in str(err.value)
    assert gpu.launch_count() == before
