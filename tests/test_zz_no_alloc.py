"""The allocation-free group collective, called through its exported C symbol.

Some users of this library cannot call cudaMalloc when they need a collective: they run
between another framework's stream-ordered work (an allocation would synchronise the
whole device), or their device memory was budgeted and reserved at start-up so a late
allocation fails.  bshmem_gpu_group_collective_noalloc keeps its per-PE table in a fixed
4 KiB array inside the library instead.  Here it is checked against the allocating entry
point on two calls in a row (the array is shared by all calls and keeps old contents, so
the second call also proves that the entry rewrites what it needs), and its size limit is
checked to fail cleanly.  Collected last on purpose: a failure here leaves every other
test already run.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _declare(lib):
    VP, I, U64 = C.c_void_p, C.c_int, C.c_uint64
    fn = lib.bshmem_gpu_group_collective_noalloc
    fn.restype = I
    fn.argtypes = [C.POINTER(VP), I, I, I, I, I, I, U64, U64, U64, I]
    lib.bshmem_gpu_noalloc_last_error.restype = C.c_char_p
    return fn


def test_noalloc_group_collective_matches_allocating_entry_twice():
    from roc_shmem_b200 import gpu
    from roc_shmem_b200.utils import dtypes as D
    group = gpu.LocalGroup(4, heap_bytes=64 << 20)
    try:
        lib = group.lib
        fn = _declare(lib)
        handles = (C.c_void_p * 4)(*[rt.h.value for rt in group.pes])
        n = 70_001
        for call, (dtype, op) in enumerate(((torch.float32, D.SUM), (torch.bfloat16, D.MAX))):
            src = group.empty((n,), dtype)
            ref = group.empty((n,), dtype)
            out = group.empty((n,), dtype)
            torch.manual_seed(10 + call)
            for s in src:
                s.copy_(torch.randn(n, device="cuda").to(dtype))
            for r, o in zip(ref, out):
                r.zero_()
                o.fill_(-1)
            torch.cuda.synchronize()
            # existing entry point (allocates its table per call)
            group.collective(gpu.COLL_REDUCE, ref, src, n, dtype=dtype, op=op, ctas=3)
            # new entry point, same arguments, through the exported C symbol
            d_off = group.pes[0].offset_of(out[0])
            s_off = group.pes[0].offset_of(src[0])
            st = fn(handles, 4, 0, gpu.COLL_REDUCE, D.code_of(dtype), op, 0, d_off, s_off, n, 3)
            assert st == 0, lib.bshmem_gpu_noalloc_last_error().decode()
            torch.cuda.synchronize()
            # plain PyTorch fp32 reference of the same reduction over the four sources
            stack = torch.stack([x.float() for x in src])
            exact = stack.sum(0) if op == D.SUM else stack.max(0).values
            for r, o in zip(ref, out):
                assert torch.allclose(o.float(), exact, rtol=2e-2 if dtype == torch.bfloat16 else 1e-5, atol=1e-5)
                assert torch.allclose(o.float(), r.float(), rtol=2e-2 if dtype == torch.bfloat16 else 1e-5, atol=1e-6)
                assert torch.equal(o, r)      # same algorithm, same order: identical bits
            if call == 1:
                # the entry allocates nothing: a repeat of the call leaves the device's free memory where it was
                free_before, _ = torch.cuda.mem_get_info()
                st = fn(handles, 4, 0, gpu.COLL_REDUCE, D.code_of(dtype), op, 0, d_off, s_off, n, 3)
                assert st == 0, lib.bshmem_gpu_noalloc_last_error().decode()
                free_after, _ = torch.cuda.mem_get_info()
                assert free_after == free_before
        # data movement through the same entry: alltoall pattern (value identifies source PE and block)
        blk = 1000
        a_src = group.empty((blk * 4,), torch.int32)
        a_dst = group.empty((blk * 4,), torch.int32)
        for i in range(4):
            for j in range(4):
                a_src[i][j * blk:(j + 1) * blk] = (i << 16) + j
        torch.cuda.synchronize()
        st = fn(handles, 4, 0, gpu.COLL_ALLTOALL, 0, 0, 0, group.pes[0].offset_of(a_dst[0]),
                group.pes[0].offset_of(a_src[0]), blk * 4, 2)
        assert st == 0, lib.bshmem_gpu_noalloc_last_error().decode()
        for i in range(4):
            for j in range(4):
                assert bool((a_dst[i][j * blk:(j + 1) * blk] == (j << 16) + i).all())
    finally:
        group.close()


def test_noalloc_rejects_ranges_outside_the_heap():
    from roc_shmem_b200 import gpu
    group = gpu.LocalGroup(2, heap_bytes=32 << 20)
    try:
        fn = _declare(group.lib)
        handles = (C.c_void_p * 2)(*[rt.h.value for rt in group.pes])
        heap = int(group.lib.bshmem_gpu_heap_bytes(group.heaps[0]))
        st = fn(handles, 2, 0, gpu.COLL_FCOLLECT, 0, 0, 0, heap - 64, 4096, 1024, 1)     # destination runs past the heap
        assert st == 4                                         # BSHMEM_ERR_RANGE, nothing was launched
        assert "outside" in group.lib.bshmem_gpu_noalloc_last_error().decode()
    finally:
        group.close()


def test_noalloc_rejects_groups_beyond_the_fixed_array():
    from roc_shmem_b200 import gpu
    group = gpu.LocalGroup(2, heap_bytes=32 << 20)
    try:
        fn = _declare(group.lib)
        too_many = (C.c_void_p * 17)(*([group.pes[0].h.value] * 17))
        st = fn(too_many, 17, 0, gpu.COLL_SYNC, 0, 0, 0, 0, 0, 0, 1)
        assert st == 6                                         # BSHMEM_ERR_LIMIT, nothing was launched
        msg = group.lib.bshmem_gpu_noalloc_last_error().decode()
        assert "16" in msg and "exceeds" in msg
    finally:
        group.close()
