"""Symmetric-heap allocator unit tests (the reference's AddressRecord / Bin / Binner /
Pow2Bins / SingleHeap gtests, clients/unit_tests/*_gtest.cpp, plus buddy coalescing)."""
import ctypes as C
import random

import pytest

from roc_shmem_b200 import _native

NO = (1 << 64) - 1


@pytest.fixture(scope="module")
def lib():
    l = _native.host_lib()
    U64, VP, I = C.c_uint64, C.c_void_p, C.c_int
    l.bshmem_unit_alloc_create.restype, l.bshmem_unit_alloc_create.argtypes = VP, [U64, U64, U64]
    l.bshmem_unit_alloc_destroy.argtypes = [VP]
    l.bshmem_unit_alloc.restype, l.bshmem_unit_alloc.argtypes = U64, [VP, U64, U64]
    l.bshmem_unit_free.restype, l.bshmem_unit_free.argtypes = I, [VP, U64]
    l.bshmem_unit_block_size.restype, l.bshmem_unit_block_size.argtypes = U64, [VP, U64]
    l.bshmem_unit_usage.argtypes = [VP, C.POINTER(U64 * 9)]
    l.bshmem_unit_roots.restype, l.bshmem_unit_roots.argtypes = I, [VP, C.POINTER(U64), C.POINTER(U64), I]
    l.bshmem_unit_round_up_pow2.restype, l.bshmem_unit_round_up_pow2.argtypes = U64, [U64, U64]
    l.bshmem_unit_record_split.argtypes = [U64, U64, C.POINTER(U64 * 4)]
    l.bshmem_unit_record_combine.restype, l.bshmem_unit_record_combine.argtypes = I, [U64, U64, U64, U64, C.POINTER(U64 * 2)]
    l.bshmem_unit_mono_create.restype, l.bshmem_unit_mono_create.argtypes = VP, [U64, U64, U64]
    l.bshmem_unit_mono_alloc.restype, l.bshmem_unit_mono_alloc.argtypes = U64, [VP, U64]
    l.bshmem_unit_mono_reset.argtypes = [VP]
    l.bshmem_unit_mono_destroy.argtypes = [VP]
    return l


def usage(lib, a):
    out = (C.c_uint64 * 9)()
    lib.bshmem_unit_usage(a, C.byref(out))
    keys = ("heap", "reserved", "allocated", "requested", "live", "largest_free", "n_allocs", "n_frees", "n_failed")
    return dict(zip(keys, (int(v) for v in out)))


def test_address_record_split_and_combine(lib):
    out = (C.c_uint64 * 4)()
    lib.bshmem_unit_record_split(1024, 512, C.byref(out))
    assert list(out) == [1024, 256, 1280, 256]
    merged = (C.c_uint64 * 2)()
    assert lib.bshmem_unit_record_combine(1024, 256, 1280, 256, C.byref(merged)) == 1 and list(merged) == [1024, 512]
    assert lib.bshmem_unit_record_combine(1280, 256, 1024, 256, C.byref(merged)) == 1 and list(merged) == [1024, 512]
    assert lib.bshmem_unit_record_combine(1024, 256, 2048, 256, C.byref(merged)) == 0      # not adjacent
    assert lib.bshmem_unit_record_combine(1024, 256, 1280, 512, C.byref(merged)) == 0      # different sizes


def test_round_up(lib):
    assert lib.bshmem_unit_round_up_pow2(1, 128) == 128
    assert lib.bshmem_unit_round_up_pow2(128, 128) == 128
    assert lib.bshmem_unit_round_up_pow2(129, 128) == 256
    assert lib.bshmem_unit_round_up_pow2((1 << 30) - 1, 128) == 1 << 30


def test_absurd_sizes_fail_fast(lib):
    """A size above 2^63 has no power of two to round up to: the request must fail, not loop (the heap lock is held)."""
    assert lib.bshmem_unit_round_up_pow2((1 << 63) + 1, 128) == 1 << 63
    a = lib.bshmem_unit_alloc_create(1 << 20, 0, 128)
    for size in ((1 << 64) - 1, (1 << 63) + 1, 1 << 62, (1 << 20) + 1):
        assert lib.bshmem_unit_alloc(a, size, 0) == NO
    assert lib.bshmem_unit_alloc(a, 1 << 20, 0) != NO                 # the heap itself still works
    lib.bshmem_unit_alloc_destroy(a)


def test_binner_roots_are_naturally_aligned(lib):
    a = lib.bshmem_unit_alloc_create(1 << 30, 4 << 20, 128)
    offs, sizes = (C.c_uint64 * 64)(), (C.c_uint64 * 64)()
    n = lib.bshmem_unit_roots(a, offs, sizes, 64)
    total = 0
    pos = 4 << 20
    for i in range(n):
        assert offs[i] == pos and offs[i] % sizes[i] == 0 and sizes[i] & (sizes[i] - 1) == 0
        pos += sizes[i]
        total += sizes[i]
    assert total == (1 << 30) - (4 << 20)
    lib.bshmem_unit_alloc_destroy(a)


def test_alloc_free_split_coalesce(lib):
    a = lib.bshmem_unit_alloc_create(1 << 20, 0, 128)
    assert lib.bshmem_unit_alloc(a, 0, 0) == NO                       # malloc(0) -> null
    x = lib.bshmem_unit_alloc(a, 100, 0)
    y = lib.bshmem_unit_alloc(a, 129, 0)
    assert x == 0 and lib.bshmem_unit_block_size(a, x) == 128
    assert y == 256 and lib.bshmem_unit_block_size(a, y) == 256       # rounded to 256, aligned to its size
    z = lib.bshmem_unit_alloc(a, 1, 0)
    assert z == 128                                                   # the split-off buddy of x is reused first
    assert lib.bshmem_unit_free(a, x) == 1 and lib.bshmem_unit_free(a, x) == 0    # double free is refused
    assert lib.bshmem_unit_free(a, 64) == 0                           # not a block start
    lib.bshmem_unit_free(a, y)
    lib.bshmem_unit_free(a, z)
    u = usage(lib, a)
    assert u["live"] == 0 and u["allocated"] == 0 and u["largest_free"] == 1 << 20   # everything coalesced back
    whole = lib.bshmem_unit_alloc(a, 1 << 20, 0)
    assert whole == 0
    assert lib.bshmem_unit_alloc(a, 128, 0) == NO                     # exhausted -> null
    assert usage(lib, a)["n_failed"] == 1
    lib.bshmem_unit_alloc_destroy(a)


def test_different_sizes_same_offsets_across_pes(lib):
    """Per-PE sizes may differ as long as they round to the same block: offsets stay symmetric
    (clients/sos_tests/asym_alloc.cpp relies on this)."""
    a = lib.bshmem_unit_alloc_create(1 << 24, 0, 128)
    b = lib.bshmem_unit_alloc_create(1 << 24, 0, 128)
    for sa, sb in ((1000, 700), (4096, 2049), (65, 128), (300000, 262145)):
        assert lib.bshmem_unit_alloc(a, sa, 0) == lib.bshmem_unit_alloc(b, sb, 0)
    lib.bshmem_unit_alloc_destroy(a)
    lib.bshmem_unit_alloc_destroy(b)


def test_alignment_and_one_gib(lib):
    a = lib.bshmem_unit_alloc_create(2 << 30, 4 << 20, 128)
    p = lib.bshmem_unit_alloc(a, 1000, 4096)
    assert p % 4096 == 0
    q = lib.bshmem_unit_alloc(a, 1 << 30, 0)
    assert q != NO and q % (1 << 30) == 0
    assert lib.bshmem_unit_alloc(a, 1 << 30, 0) == NO
    lib.bshmem_unit_alloc_destroy(a)


def test_random_alloc_free_never_overlaps_and_is_deterministic(lib):
    def run(seed):
        rng = random.Random(seed)
        a = lib.bshmem_unit_alloc_create(8 << 20, 1 << 16, 128)
        live = {}
        trace = []
        for _ in range(3000):
            if live and rng.random() < 0.45:
                off = rng.choice(list(live))
                assert lib.bshmem_unit_free(a, off) == 1
                del live[off]
            else:
                size = rng.choice([1, 100, 128, 1000, 5000, 70000, 300000])
                off = lib.bshmem_unit_alloc(a, size, 0)
                trace.append(off)
                if off != NO:
                    blk = lib.bshmem_unit_block_size(a, off)
                    assert blk >= size and off % blk == 0 and off >= (1 << 16)
                    for o, b in live.items():
                        assert off + blk <= o or o + b <= off, "blocks overlap"
                    live[off] = blk
        for off in list(live):
            lib.bshmem_unit_free(a, off)
        assert usage(lib, a)["allocated"] == 0
        lib.bshmem_unit_alloc_destroy(a)
        return trace
    assert run(7) == run(7)


def test_mono_linear(lib):
    m = lib.bshmem_unit_mono_create(4096, 1024, 128)
    assert lib.bshmem_unit_mono_alloc(m, 100) == 4096
    assert lib.bshmem_unit_mono_alloc(m, 1) == 4096 + 128
    assert lib.bshmem_unit_mono_alloc(m, 2000) == NO
    lib.bshmem_unit_mono_reset(m)
    assert lib.bshmem_unit_mono_alloc(m, 1024) == 4096
    lib.bshmem_unit_mono_destroy(m)
