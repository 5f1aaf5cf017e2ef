"""NVLink runtime on one GPU: a 1-PE job through the public init path, and a
4-PE "local group" whose collectives run as one cooperative launch."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    import roc_shmem_b200 as shmem
    r = shmem.init("device", rank=0, world_size=1, heap_bytes=256 << 20, timeout_ms=2000)
    yield r
    shmem.finalize()


def test_single_pe_put_get_roundtrip(rt):
    x = rt.empty((1 << 16,), torch.float32)
    src = torch.randn(1 << 16, device="cuda")
    rt.put(x, src, 0)
    rt.quiet()
    assert torch.equal(x, src)
    back = torch.empty_like(src)
    rt.get(back, x, 0)
    assert torch.equal(back, src)
    host = torch.arange(1 << 16, dtype=torch.float32)          # host source buffers are allowed
    rt.put(x, host, 0)
    assert torch.equal(x.cpu(), host)
    rt.free(x)


def test_single_pe_atomics(rt):
    c = rt.zeros((2,), torch.int64)
    assert rt.atomic_fetch_add(c, 5, 0) == 0
    assert rt.atomic_fetch_inc(c, 0) == 5
    assert rt.atomic_fetch(c, 0) == 6
    assert rt.atomic_compare_swap(c, 6, 42, 0) == 6
    assert rt.atomic_swap(c, 7, 0) == 42
    rt.atomic_add(c, 3, 0)
    rt.atomic_inc(c, 0)
    rt.atomic_set(c[1:], 0xF0, 0)
    assert rt.atomic_fetch_and(c[1:], 0x3C, 0) == 0xF0
    assert rt.atomic_fetch_or(c[1:], 0x03, 0) == 0x30
    assert rt.atomic_fetch_xor(c[1:], 0xFF, 0) == 0x33
    rt.quiet()
    assert c.tolist() == [11, 0xCC]
    f = rt.zeros((1,), torch.float32)
    assert rt.atomic_fetch_add(f, 1.5, 0) == 0.0
    assert rt.atomic_swap(f, 4.0, 0) == 1.5
    rt.free(f)
    rt.free(c)


def test_single_pe_signal_wait_and_timeout(rt):
    import roc_shmem_b200 as shmem
    data = rt.empty((1024,), torch.int32)
    sig = rt.zeros((1,), torch.int64)
    src = torch.arange(1024, device="cuda", dtype=torch.int32)
    rt.put_signal(data, src, sig, 7, 0)
    rt.wait_until(sig, "eq", 7)
    assert torch.equal(data, src)
    assert rt.test(sig, "ge", 7) and not rt.test(sig, "gt", 7)
    # a flag nobody sets: the bounded device wait must come back with a timeout status
    from roc_shmem_b200.utils.timeouts import temporary_timeout
    never = rt.zeros((1,), torch.int64)
    with temporary_timeout(rt, 50):
        with pytest.raises(shmem.ShmemTimeout):
            rt.wait_until(never, "eq", 1)
    rec = rt.error_record()
    assert rec["code"] == 3 and rec["where"] == 1
    # the context is still usable afterwards
    rt.put(data, src + 1, 0)
    assert torch.equal(data, src + 1)


def test_single_pe_collectives_and_device_rma(rt):
    a = rt.empty((4096,), torch.float32)
    b = rt.empty((4096,), torch.float32)
    a.copy_(torch.randn(4096, device="cuda"))
    rt.barrier_all()
    rt.reduce(b, a, "sum")
    rt.quiet()
    assert torch.equal(a, b)
    big = rt.empty((8 << 20,), torch.uint8)
    src = torch.randint(0, 255, (8 << 20,), device="cuda", dtype=torch.uint8)
    for scope in ("block", "warp", "thread"):
        big.zero_()
        rt.rma_kernel(big, src, 0, put=True, scope=scope, ctas=16, threads=256)
        rt.quiet()
        assert torch.equal(big, src), scope
    out = torch.zeros_like(src)
    rt.rma_kernel(big, out, 0, put=False, scope="block", ctas=16)
    rt.quiet()
    assert torch.equal(out, src)
    st = rt.device_stats()
    assert st["put"] > 0 and st["bytes_put"] >= 3 * (8 << 20)


@pytest.fixture(scope="module")
def group():
    from roc_shmem_b200.gpu import LocalGroup
    g = LocalGroup(4, heap_bytes=64 << 20)
    yield g
    g.close()


def test_group_host_put_reaches_peer_heap(group):
    xs = group.empty((1000,), torch.int32)
    for x in xs:
        x.zero_()
    src = torch.arange(1000, device="cuda", dtype=torch.int32)
    group.pes[0].put(xs[0], src, 2)          # PE 0 writes into PE 2's copy
    group.pes[0].quiet()
    assert torch.equal(xs[2], src) and int(xs[0].sum()) == 0 and int(xs[1].sum()) == 0
    # a PE always names the target by its OWN symmetric address plus the target PE number
    assert group.pes[3].atomic_fetch_add(xs[3], 9, 1) == 0
    assert int(xs[1][0]) == 9 and int(xs[3][0]) == 0


@pytest.mark.parametrize("dtype,n", [(torch.float32, 1000), (torch.float32, 300_000), (torch.bfloat16, 65_536),
                                     (torch.int64, 4097), (torch.float16, 12_345)])
def test_group_allreduce_sum(group, dtype, n):
    from roc_shmem_b200 import gpu
    srcs = group.empty((n,), dtype)
    dsts = group.empty((n,), dtype)
    torch.manual_seed(1)
    for i, s in enumerate(srcs):
        if dtype.is_floating_point:
            s.copy_(torch.randn(n, device="cuda").to(dtype))
        else:
            s.copy_(torch.randint(-1000, 1000, (n,), device="cuda", dtype=dtype))
    group.collective(gpu.COLL_REDUCE, dsts, srcs, n, dtype=dtype, op=0, ctas=3)
    if dtype.is_floating_point:
        acc = srcs[0].float()
        for s in srcs[1:]:
            acc = acc + s.float()
        ref = acc.to(dtype)
    else:
        ref = sum(srcs[1:], srcs[0].clone())
    for d in dsts:
        assert torch.equal(d, ref)


def test_group_allreduce_in_place_max(group):
    from roc_shmem_b200 import gpu
    n = 50_000
    bufs = group.empty((n,), torch.float32)
    vals = [torch.randn(n, device="cuda") for _ in bufs]
    for b, v in zip(bufs, vals):
        b.copy_(v)
    group.collective(gpu.COLL_REDUCE, bufs, bufs, n, dtype=torch.float32, op=2, ctas=2)
    ref = torch.stack(vals).max(dim=0).values
    for b in bufs:
        assert torch.equal(b, ref)


def test_group_broadcast_fcollect_alltoall_reduce_scatter(group):
    from roc_shmem_b200 import gpu
    P = group.n_pes
    n = 10_000
    src = group.empty((n,), torch.int32)
    dst = group.empty((n,), torch.int32)
    for i in range(P):
        src[i].fill_(i + 1)
        dst[i].fill_(-1)
    group.collective(gpu.COLL_BROADCAST, dst, src, n * 4, root=2, ctas=2)
    for i in range(P):
        assert bool((dst[i] == (-1 if i == 2 else 3)).all())      # the root's dest stays untouched

    fd = group.empty((n * P,), torch.int32)
    group.collective(gpu.COLL_FCOLLECT, fd, src, n * 4, ctas=2)
    for i in range(P):
        for j in range(P):
            assert bool((fd[i][j * n:(j + 1) * n] == j + 1).all())

    a_src = group.empty((n * P,), torch.int32)
    a_dst = group.empty((n * P,), torch.int32)
    for i in range(P):
        for j in range(P):
            a_src[i][j * n:(j + 1) * n] = (i << 16) + j       # value identifies (source PE, block)
    group.collective(gpu.COLL_ALLTOALL, a_dst, a_src, n * 4, ctas=2)
    for i in range(P):
        for j in range(P):
            assert bool((a_dst[i][j * n:(j + 1) * n] == (j << 16) + i).all())

    rs_src = group.empty((n * P,), torch.float32)
    rs_dst = group.empty((n,), torch.float32)
    for i in range(P):
        rs_src[i].copy_(torch.randn(n * P, device="cuda"))
    group.collective(gpu.COLL_REDUCE_SCATTER, rs_dst, rs_src, n, dtype=torch.float32, op=0, ctas=2)
    for i in range(P):
        acc = rs_src[0][i * n:(i + 1) * n].clone()
        for k in range(1, P):
            acc = acc + rs_src[k][i * n:(i + 1) * n]
        assert torch.equal(rs_dst[i], acc)


def test_group_rooted_reduce(group):
    """Rooted reduce: the root's dest gets the float32 sum of every PE's source in PE order, the others stay as they were;
    small (one block) and large (several blocks, bulk path) vectors."""
    from roc_shmem_b200 import gpu
    P = group.n_pes
    for n, ctas in ((1000, 1), (3_000_000, 8)):
        src = group.empty((n,), torch.float32)
        dst = group.empty((n,), torch.float32)
        for i in range(P):
            src[i].copy_(torch.randn(n, device="cuda"))
            dst[i].fill_(-3.0)
        group.collective(gpu.COLL_REDUCE_ROOT, dst, src, n, dtype=torch.float32, op=0, root=1, ctas=ctas)
        acc = src[0].clone()
        for k in range(1, P):
            acc = acc + src[k]
        for i in range(P):
            assert torch.equal(dst[i], acc) if i == 1 else bool((dst[i] == -3.0).all())


def test_group_team_split_and_team_reduce(group):
    from roc_shmem_b200 import gpu
    slots = group.team_split(0, 0, 2, 2)                  # PEs {0, 2}
    assert slots[0] == slots[2] > 0 and slots[1] == -1 and slots[3] == -1
    n = 2048
    src = group.empty((n,), torch.float32)
    dst = group.empty((n,), torch.float32)
    for i in range(group.n_pes):
        src[i].fill_(float(i + 1))
        dst[i].zero_()
    group.collective(gpu.COLL_REDUCE, dst, src, n, dtype=torch.float32, op=0, team_slot=slots[0], ctas=1)
    assert bool((dst[0] == 4).all()) and bool((dst[2] == 4).all())
    assert bool((dst[1] == 0).all()) and bool((dst[3] == 0).all())
    # back-to-back collectives on the same team reuse the epoch flags safely
    for _ in range(5):
        group.collective(gpu.COLL_REDUCE, dst, src, n, dtype=torch.float32, op=0, team_slot=slots[0], ctas=1)
    assert bool((dst[0] == 4).all())


@pytest.mark.parametrize("scope", ["thread", "warp", "block"])
@pytest.mark.parametrize("put", [True, False])
def test_device_rma_matrix_sizes_and_alignments(rt, scope, put):
    """The reference's functional sweep (clients/functional_tests/driver.sh:62-86: one work-group of 64 threads and
    25 work-groups of 1024 threads, sizes in powers of two) plus odd sizes and misaligned ends, checked byte-exactly
    with guard bytes on both sides."""
    sym = rt.empty((1 << 20,), torch.uint8)
    local = torch.empty(1 << 20, dtype=torch.uint8, device="cuda")
    pattern = (torch.arange(1 << 20, device="cuda") * 7 + 3).to(torch.uint8)
    for ctas, threads in ((1, 64), (25, 1024)):
        for nbytes in (1, 2, 4, 8, 15, 16, 64, 100, 1024, 4097, 32768, 65536 + 5, (1 << 19) + 13):
            for off_sym, off_loc in ((0, 0), (1, 1), (16, 3), (5, 64)):
                if nbytes > 4096 and (off_sym, off_loc) == (16, 3) and scope == "thread":
                    continue                                   # keep the byte-wise single-thread path short
                s = sym[256 + off_sym:256 + off_sym + nbytes]
                l = local[256 + off_loc:256 + off_loc + nbytes]
                if put:
                    sym.fill_(0xEE)
                    local.copy_(pattern)
                else:
                    sym.copy_(pattern)
                    local.fill_(0xEE)
                rt.rma_kernel(s, l, 0, put=put, scope=scope, ctas=ctas, threads=threads, nbytes=nbytes)
                rt.quiet()
                dst, src, o_dst, o_src = (sym, pattern, off_sym, off_loc) if put else (local, pattern, off_loc, off_sym)
                lo, hi = 256 + o_dst, 256 + o_dst + nbytes
                assert torch.equal(dst[lo:hi], src[256 + o_src:256 + o_src + nbytes]), (scope, put, ctas, nbytes, off_sym, off_loc)
                assert bool((dst[:lo] == 0xEE).all()) and bool((dst[hi:] == 0xEE).all()), "guard bytes touched"
    rt.free(sym)


def test_device_timeline_records_puts_and_waits(rt):
    """The event ring behind the device counters: off by default, keeps the last `capacity` events in order."""
    sym = rt.zeros((1 << 16,), torch.uint8)
    src = torch.ones(1 << 16, dtype=torch.uint8, device="cuda")
    rt.trace_enable(0)
    rt.rma_kernel(sym, src, 0, put=True, scope="block", ctas=4, threads=128)
    rt.quiet()
    assert rt.trace_events() == []
    rt.trace_enable(8)
    rt.rma_kernel(sym, src, 0, put=True, scope="block", ctas=4, threads=128)       # 4 put events (one per CTA)
    rt.rma_kernel(sym, src, 0, put=False, scope="block", ctas=2, threads=128)      # 2 get events
    rt.quiet()
    ev = rt.trace_events()
    assert [e["op"] for e in ev].count("put") == 4 and [e["op"] for e in ev].count("get") == 2
    assert sorted(e["block"] for e in ev if e["op"] == "put") == [0, 1, 2, 3]
    assert all(e["pe"] == 0 and e["bytes"] == (1 << 16) // (4 if e["op"] == "put" else 2) for e in ev)
    assert [e["seq"] for e in ev] == list(range(6)) and all(ev[i]["t_ns"] <= ev[i + 1]["t_ns"] + 10_000_000 for i in range(5))
    for _ in range(3):                                                             # overflow: the ring keeps the last 8
        rt.rma_kernel(sym, src, 0, put=True, scope="block", ctas=4, threads=128)
    rt.quiet()
    ev = rt.trace_events()
    assert len(ev) == 8 and [e["seq"] for e in ev] == list(range(10, 18))
    rt.trace_enable(0)
    rt.free(sym)


@pytest.mark.parametrize("dtype,n,op", [(torch.float32, 1000, 0), (torch.float32, 1, 2), (torch.bfloat16, 2048, 0),
                                        (torch.int64, 512, 0), (torch.int32, 77, 1), (torch.float64, 33, 3)])
def test_group_allreduce_low_latency_path(group, dtype, n, op):
    """Vectors of at most 4 KiB on the world team with one block take the one-exchange path (data and epoch in the
    same 8-byte store); repeated calls alternate the slot parity, the last call reduces in place."""
    from roc_shmem_b200 import gpu
    srcs = group.empty((n,), dtype)
    dsts = group.empty((n,), dtype)
    torch.manual_seed(n)
    for rep in range(5):
        for s in srcs:
            if dtype.is_floating_point:
                s.copy_((torch.rand(n, device="cuda") + 0.5).to(dtype))
            else:
                s.copy_(torch.randint(1, 5, (n,), device="cuda", dtype=dtype))
        wide = torch.float64 if dtype.is_floating_point else torch.int64
        st = torch.stack([s.to(wide) for s in srcs])
        ref = (st.sum(0) if op == 0 else st.min(0).values if op == 1 else st.max(0).values if op == 2 else st.prod(0))
        in_place = rep == 4
        group.collective(gpu.COLL_REDUCE, srcs if in_place else dsts, srcs, n, dtype=dtype, op=op, ctas=1)
        for d in (srcs if in_place else dsts):
            if dtype.is_floating_point:
                assert torch.allclose(d.to(wide), ref, rtol=2e-2 if dtype == torch.bfloat16 else 1e-6), (rep, dtype)
            else:
                assert torch.equal(d.to(wide), ref), (rep, dtype)


def test_group_team_allreduce_low_latency_path(group):
    """Teams other than the world team have their own one-exchange slots (vectors of at most 1 KiB, one block);
    two disjoint teams use theirs independently and repeated calls alternate the slot parity."""
    from roc_shmem_b200 import gpu
    even = group.team_split(0, 0, 2, 2)                   # PEs {0, 2}
    odd = group.team_split(0, 1, 2, 2)                    # PEs {1, 3}
    assert even[0] == even[2] > 0 and odd[1] == odd[3] > 0 and even[0] != odd[1]
    n = 200
    src = group.empty((n,), torch.float32)
    dst = group.empty((n,), torch.float32)
    dst2 = group.empty((n,), torch.float32)
    # a slot number means "my team in that slot" on every PE, and PEs outside a team may hold an older team under the
    # same number, so each team's result goes to its own buffer and only its members' copies are checked
    for rep in range(6):
        for i in range(group.n_pes):
            src[i].copy_(torch.arange(n, device="cuda", dtype=torch.float32) + 10 * i + rep)
            dst[i].zero_()
            dst2[i].zero_()
        group.collective(gpu.COLL_REDUCE, dst, src, n, dtype=torch.float32, op=0, team_slot=even[0], ctas=1)
        group.collective(gpu.COLL_REDUCE, dst2, src, n, dtype=torch.float32, op=2, team_slot=odd[1], ctas=1)
        base = torch.arange(n, device="cuda", dtype=torch.float32) + rep
        assert torch.equal(dst[0], 2 * base + 20) and torch.equal(dst[2], 2 * base + 20)      # sum over PEs 0 and 2
        assert torch.equal(dst2[1], base + 30) and torch.equal(dst2[3], base + 30)            # max over PEs 1 and 3
