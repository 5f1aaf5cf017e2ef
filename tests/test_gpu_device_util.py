"""Device utilities: block mutexes (counter == blocks * iterations), slab allocator, notifier,
index strategies (every element visited the expected number of times), warp-aggregated sharing,
and the warp coalescer's merge rule."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    from roc_shmem_b200.gpu import cuda_lib
    lib = cuda_lib()
    VP, I, U64 = C.c_void_p, C.c_int, C.c_uint64
    lib.bshmem_util_scratch_bytes.restype = I
    lib.bshmem_util_init.argtypes = [VP, VP, U64]
    lib.bshmem_util_mutex_test.argtypes = [VP, I, I, I, I, I, C.POINTER(U64), C.POINTER(I)]
    lib.bshmem_util_slab_test.argtypes = [VP, I, I, I, VP, I, C.POINTER(I)]
    lib.bshmem_util_index_test.argtypes = [I, I, I, VP, U64]
    lib.bshmem_util_share_test.argtypes = [VP, I, I, VP]
    lib.bshmem_util_coalesce_test.argtypes = [VP, VP, I, VP, VP]
    scratch = torch.zeros(lib.bshmem_util_scratch_bytes() + 256, dtype=torch.uint8, device="cuda")
    slab = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    sp = (scratch.data_ptr() + 255) // 256 * 256
    assert lib.bshmem_util_init(sp, slab.data_ptr(), slab.numel()) == 0
    return lib, sp, slab, scratch


@pytest.mark.parametrize("which", [0, 1])
def test_block_mutex_counts_every_entry(env, which):
    lib, sp, slab, _ = env
    assert lib.bshmem_util_init(sp, slab.data_ptr(), slab.numel()) == 0
    counter, status = C.c_uint64(0), C.c_int(0)
    blocks, iters = 24, 20           # at most 32 waiters at once for the 32-slot queue lock
    assert lib.bshmem_util_mutex_test(sp, which, blocks, 128, iters, 5000, C.byref(counter), C.byref(status)) == 0
    assert status.value == 0 and counter.value == blocks * iters


def test_slab_heap_block_allocations(env):
    lib, sp, slab, _ = env
    assert lib.bshmem_util_init(sp, slab.data_ptr(), slab.numel()) == 0
    blocks, allocs = 16, 5
    offs = torch.zeros(blocks * allocs, dtype=torch.int64, device="cuda")
    status = C.c_int(0)
    assert lib.bshmem_util_slab_test(sp, blocks, 96, allocs, offs.data_ptr(), 5000, C.byref(status)) == 0
    assert status.value == 0
    o = offs.view(blocks, allocs).cpu()
    spans = sorted((int(o[b, a]), (b + 1) * 64, b + 1) for b in range(blocks) for a in range(allocs))
    data = slab.cpu()
    for (start, size, owner), nxt in zip(spans, spans[1:] + [(1 << 20, 0, 0)]):
        assert start % 128 == 0 and start + size <= nxt[0]                 # aligned, no overlap
        assert bool((data[start:start + size] == owner).all())               # written by the block that got it


def test_index_strategies_visit_counts(env):
    lib = env[0]
    n, blocks, threads = 10_007, 4, 128
    expect = {0: blocks * threads, 1: blocks, 2: blocks, 3: blocks * threads // 32, 4: 1, 5: 1, 6: blocks}
    for strategy, per_elem in expect.items():
        visits = torch.zeros(n, dtype=torch.int32, device="cuda")
        assert lib.bshmem_util_index_test(strategy, blocks, threads, visits.data_ptr(), n) == 0
        assert bool((visits == per_elem).all()), strategy


def test_share_strategy_hands_out_distinct_values(env):
    lib, sp, slab, _ = env
    assert lib.bshmem_util_init(sp, slab.data_ptr(), slab.numel()) == 0
    blocks, threads = 8, 256
    t = torch.zeros(blocks * threads, dtype=torch.int64, device="cuda")
    assert lib.bshmem_util_share_test(sp, blocks, threads, t.data_ptr()) == 0
    got = t.cpu()
    taken = got[got >= 0]
    assert taken.numel() == blocks * threads // 2 and sorted(taken.tolist()) == list(range(blocks * threads // 2))


def test_warp_coalescer_merges_contiguous_lanes(env):
    lib = env[0]
    size = 64
    pes = torch.zeros(32, dtype=torch.int32, device="cuda")
    offs = torch.arange(32, dtype=torch.int64, device="cuda") * size      # all 32 lanes contiguous
    send = torch.zeros(32, dtype=torch.int32, device="cuda")
    out = torch.zeros(32, dtype=torch.int64, device="cuda")
    assert lib.bshmem_util_coalesce_test(pes.data_ptr(), offs.data_ptr(), size, send.data_ptr(), out.data_ptr()) == 0
    assert send.tolist() == [1] + [0] * 31 and int(out[0]) == 32 * size
    # a gap after lane 7, another PE from lane 16, lane 20 inactive
    offs2 = offs.clone()
    offs2[8:] += 4096
    pes[16:] = 1
    offs2[20] = -1
    assert lib.bshmem_util_coalesce_test(pes.data_ptr(), offs2.data_ptr(), size, send.data_ptr(), out.data_ptr()) == 0
    s, o = send.tolist(), out.tolist()
    heads = [i for i, v in enumerate(s) if v == 1]
    assert heads == [0, 8, 16, 21] and s[20] == -1
    assert [o[h] for h in heads] == [8 * size, 8 * size, 4 * size, 11 * size]
