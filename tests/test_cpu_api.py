"""Host API on the CPU backend (PE threads over a shared heap): the reference's host test
programs (clients/sos_tests/*.cpp) re-expressed with closed-form checks."""
import ctypes as C
import math

import pytest
import torch

import roc_shmem_b200 as shmem
from roc_shmem_b200.config import Config
from roc_shmem_b200.cpu import run_threads
from roc_shmem_b200.utils.timeouts import temporary_timeout


def test_hello_and_queries():
    def body(rt):
        assert rt.n_pes == 3 and 0 <= rt.my_pe < 3
        assert rt.query_thread() == 4                      # THREAD_MULTIPLE
        assert rt.team_world.n_pes == 3 and rt.team_world.my_pe == rt.my_pe
        return rt.my_pe
    assert run_threads(3, body, heap_bytes=1 << 20) == [0, 1, 2]


def test_put_get_p_g_typed():
    def body(rt):
        me, n = rt.my_pe, rt.n_pes
        for dtype in (torch.int8, torch.int16, torch.int32, torch.int64, torch.uint8, torch.float32, torch.float64,
                      torch.bfloat16, torch.float16):
            sym = rt.empty((257,), dtype)
            sym.zero_()
            rt.barrier_all()
            src = (torch.arange(257) % 100 + me).to(dtype)
            rt.put(sym, src, (me + 1) % n)
            rt.barrier_all()
            assert torch.equal(sym, (torch.arange(257) % 100 + (me - 1) % n).to(dtype)), dtype
            got = torch.empty(257, dtype=dtype)
            rt.get(got, sym, (me + 1) % n)
            assert torch.equal(got, src), dtype
            rt.barrier_all()
            rt.p(sym, 7, (me + 1) % n)
            rt.barrier_all()
            assert rt.g(sym, me) == 7 and rt.g(sym, (me + 1) % n) == 7
            rt.free(sym)
    run_threads(2, body, heap_bytes=4 << 20)


def test_zero_length_and_bad_arguments():
    def body(rt):
        sym = rt.empty((16,), torch.int32)
        rt.put(sym, torch.empty(0, dtype=torch.int32), 0)              # zero-length ops are no-ops
        with pytest.raises(shmem.ShmemError):
            rt.put(sym, torch.zeros(16, dtype=torch.int32), 99)        # PE out of range
        with pytest.raises(shmem.ShmemError):
            rt.put(torch.zeros(16, dtype=torch.int32), sym, 0)         # dest is not symmetric
        with pytest.raises(shmem.ShmemError):
            rt.put(sym, torch.zeros(1 << 22, dtype=torch.int32), 0)    # runs off the heap
        assert rt.ptr(sym, 0) != 0 and rt.ptr(torch.zeros(1), 0) == 0
        rt.barrier_all()
    run_threads(2, body, heap_bytes=1 << 20)


def test_atomics_closed_form():
    def body(rt):
        me, n = rt.my_pe, rt.n_pes
        c = rt.zeros((4,), torch.int64)
        for _ in range(100):
            rt.atomic_add(c, 3, 0)
            rt.atomic_inc(c[1:], 0)
        old = [rt.atomic_fetch_inc(c[2:], 0) for _ in range(50)]
        rt.barrier_all()
        if me == 0:
            assert c[:3].tolist() == [300 * n, 100 * n, 50 * n]
        assert len(set(old)) == 50
        rt.barrier_all()
        # compare-and-swap election: exactly one PE wins
        won = rt.atomic_compare_swap(c[3:], 0, me + 1, 0) == 0
        rt.barrier_all()
        winner = rt.atomic_fetch(c[3:], 0)
        assert (winner == me + 1) == won
        rt.barrier_all()
        u = rt.zeros((1,), torch.int32)
        if me == 0:
            rt.atomic_set(u, 0xF0, 1)
            assert rt.atomic_fetch_and(u, 0x3C, 1) == 0xF0
            assert rt.atomic_fetch_or(u, 0x03, 1) == 0x30
            assert rt.atomic_fetch_xor(u, 0xFF, 1) == 0x33
            rt.atomic_and(u, 0xF0, 1); rt.atomic_or(u, 0x01, 1); rt.atomic_xor(u, 0x10, 1)
            assert rt.atomic_swap(u, 5, 1) == 0xD1
        rt.barrier_all()
        if me == 1:
            assert int(u[0]) == 5
        f = rt.zeros((1,), torch.float64)
        rt.atomic_add(f, 0.5, 0)
        rt.barrier_all()
        assert rt.atomic_fetch(f, 0) == 0.5 * n
        g = rt.zeros((1,), torch.float32)
        assert rt.atomic_swap(g, 2.5, me) == 0.0 and rt.atomic_fetch(g, me) == 2.5
        rt.barrier_all()
        return won
    res = run_threads(3, body, heap_bytes=1 << 20)
    assert sum(res) == 1


def test_wait_until_test_and_signal():
    def body(rt):
        me, n = rt.my_pe, rt.n_pes
        flag = rt.zeros((1,), torch.int32)
        data = rt.zeros((256,), torch.float32)
        sig = rt.zeros((1,), torch.int64)
        if me == 0:
            for pe in range(1, n):
                rt.put(data, torch.full((256,), 3.5), pe)
                rt.fence()
                rt.p(flag, 1, pe)
        else:
            assert rt.test(flag, "eq", 0) in (True, False)
            rt.wait_until(flag, "ne", 0)
            assert bool((data == 3.5).all())               # put + fence + flag ordering
            for cmp, val, ok in (("eq", 1, True), ("ne", 1, False), ("gt", 0, True), ("ge", 1, True), ("lt", 2, True),
                                 ("le", 0, False)):
                assert rt.test(flag, cmp, val) == ok
        rt.barrier_all()
        rt.put_signal(data, torch.full((256,), float(me)), sig, 5, (me + 1) % n, op=1)   # SIGNAL_ADD
        rt.wait_until(sig, "eq", 5)
        assert bool((data == float((me - 1) % n)).all())
        assert rt.signal_fetch(sig) == 5
        rt.barrier_all()
    run_threads(3, body, heap_bytes=1 << 20)


@pytest.mark.parametrize("dtype", [torch.int16, torch.int32, torch.int64, torch.float32, torch.float64, torch.bfloat16])
def test_to_all_every_op(dtype):
    def body(rt):
        me, n = rt.my_pe, rt.n_pes
        src = rt.empty((1000,), dtype)
        dst = rt.empty((1000,), dtype)
        vals = (torch.arange(1000) % 7 + me + 1).to(dtype)
        ops = ["sum", "min", "max", "prod"] + ([] if dtype.is_floating_point else ["and", "or", "xor"])
        for op in ops:
            src.copy_(vals)
            rt.reduce(dst, src, op)
            cols = [(torch.arange(1000) % 7 + p + 1) for p in range(n)]
            st = torch.stack(cols)
            if op == "sum": ref = st.sum(0)
            elif op == "min": ref = st.min(0).values
            elif op == "max": ref = st.max(0).values
            elif op == "prod": ref = st.prod(0)
            elif op == "and": ref = cols[0] & cols[1] & cols[2]
            elif op == "or": ref = cols[0] | cols[1] | cols[2]
            else: ref = cols[0] ^ cols[1] ^ cols[2]
            assert torch.equal(dst, ref.to(dtype)), (dtype, op)
        src.copy_(vals)
        rt.reduce(src, src, "sum")                          # reduce in place
        assert torch.equal(src, torch.stack([(torch.arange(1000) % 7 + p + 1) for p in range(n)]).sum(0).to(dtype))
    run_threads(3, body, heap_bytes=1 << 20)


def test_bitwise_reduction_on_float_is_rejected():
    def body(rt):
        s = rt.empty((8,), torch.float32)
        with pytest.raises(shmem.ShmemError):
            rt.reduce(s, s, "xor")
    run_threads(1, body, heap_bytes=1 << 20)


def test_broadcast_fcollect_alltoall_reduce_scatter():
    def body(rt):
        me, n = rt.my_pe, rt.n_pes
        src = rt.empty((100,), torch.int64)
        dst = rt.empty((100,), torch.int64)
        src.fill_(me + 1)
        dst.fill_(-1)
        rt.broadcast(dst, src, 1)
        assert bool((dst == (-1 if me == 1 else 2)).all())          # the root's dest is not written
        big = rt.empty((100 * n,), torch.int64)
        rt.fcollect(big, src)
        assert big.view(n, 100)[:, 0].tolist() == [p + 1 for p in range(n)]
        a_src = rt.empty((100 * n,), torch.int64)
        for j in range(n):
            a_src[j * 100:(j + 1) * 100] = (me << 16) + j
        rt.alltoall(big, a_src)
        assert big.view(n, 100)[:, 0].tolist() == [(j << 16) + me for j in range(n)]
        rs = rt.empty((100,), torch.int64)
        rt.reduce_scatter(rs, a_src, "sum")
        assert bool((rs == sum((p << 16) + me for p in range(n))).all())
    run_threads(4, body, heap_bytes=1 << 20)


def test_collectives_with_eight_and_sixteen_pes():
    """The host runtime at the PE counts of a full node: world collectives, a strided team of every other PE and a
    team-relative context, with 8 and with 16 (= BSHMEM_MAX_PES) PEs."""
    def body(rt):
        me, n = rt.my_pe, rt.n_pes
        src = rt.empty((33,), torch.int64)
        src.fill_(me + 1)
        big = rt.empty((33 * n,), torch.int64)
        rt.fcollect(big, src)
        assert big.view(n, 33)[:, 7].tolist() == [p + 1 for p in range(n)]
        a_src = rt.empty((33 * n,), torch.int64)
        for j in range(n):
            a_src[j * 33:(j + 1) * 33] = (me << 16) + j
        rt.alltoall(big, a_src)
        assert big.view(n, 33)[:, 0].tolist() == [(j << 16) + me for j in range(n)]
        acc = rt.empty((33,), torch.int64)
        rt.reduce(acc, src, "sum")
        assert bool((acc == n * (n + 1) // 2).all())
        rt.reduce_scatter(acc, a_src, "max")
        assert bool((acc == ((n - 1) << 16) + me).all())
        acc.fill_(-1)
        rt.reduce_root(acc, src, n - 1, "sum")
        assert bool((acc == (n * (n + 1) // 2 if me == n - 1 else -1)).all())
        rt.barrier_all()
        even = rt.team_split_strided(None, 0, 2, n // 2)
        if even.valid:
            assert even.n_pes == n // 2 and even.my_pe == me // 2
        f = rt.empty((4,), torch.float32)
        g = rt.zeros((4,), torch.float32)
        f.fill_(float(me))
        if even.valid:
            rt.reduce(g, f, "sum", team=even)
            assert bool((g == float(sum(range(0, n, 2)))).all())
            even.sync()                                        # every member has its result before anyone overwrites g[0]
            with rt.ctx_create(0, even) as c:
                c.put(g[:1], torch.tensor([1000.0 + me]), (even.my_pe + 1) % even.n_pes)   # team-relative neighbour
            even.sync()
            assert float(g[0]) == 1000.0 + (me - 2) % n
            even.destroy()
        rt.barrier_all()
    run_threads(8, body, heap_bytes=1 << 20)
    run_threads(16, body, heap_bytes=1 << 20)


def test_rooted_reduce():
    """Only the root's dest receives the reduction; a sub-team numbers its root relative to the team."""
    def body(rt):
        me, n = rt.my_pe, rt.n_pes
        src = rt.empty((64,), torch.int32)
        dst = rt.empty((64,), torch.int32)
        src.copy_(torch.arange(64, dtype=torch.int32) + 10 * me)
        dst.fill_(-7)
        rt.reduce_root(dst, src, 2, "sum")
        want = torch.arange(64, dtype=torch.int32) * n + 10 * sum(range(n))
        assert torch.equal(dst, want) if me == 2 else bool((dst == -7).all())
        rt.barrier_all()
        rt.reduce_root(src, src, 0, "max")                           # in place on the root
        if me == 0:
            assert torch.equal(src, torch.arange(64, dtype=torch.int32) + 10 * (n - 1))
        else:
            assert torch.equal(src, torch.arange(64, dtype=torch.int32) + 10 * me)
        rt.barrier_all()
        odd = rt.team_world.split_strided(1, 2, n // 2)              # PEs 1, 3
        f = rt.empty((8,), torch.float32)                            # symmetric allocations are collective over the world
        g = rt.zeros((8,), torch.float32)
        f.fill_(float(me))
        if me % 2 == 1:
            rt.reduce_root(g, f, 1, "sum", team=odd)                 # team member 1 = PE 3
            assert bool((g == (4.0 if me == 3 else 0.0)).all())
            with pytest.raises(shmem.ShmemError):
                rt.reduce_root(g, f, 2, "sum", team=odd)             # not a member
    run_threads(4, body, heap_bytes=1 << 20)


def test_active_set_forms():
    def body(rt):
        me, n = rt.my_pe, rt.n_pes
        psync = rt.zeros((256,), torch.int64)
        src = rt.empty((64,), torch.int32)
        dst = rt.zeros((64,), torch.int32)
        src.fill_(me + 1)
        rt.barrier_all()
        if me % 2 == 0:                                            # active set: PEs 0, 2 (start 0, stride 2^1, size 2)
            for _ in range(3):
                rt.barrier_active_set(0, 1, 2, psync)
            rt.to_all_active_set(dst, src, "sum", 0, 1, 2, None, psync)
            assert bool((dst == 1 + 3).all())
            rt.broadcast_active_set(dst, src, 1, 0, 1, 2, psync)   # root index 1 of the set = PE 2
            assert bool((dst == (4 if me == 2 else 3)).all())
            assert bool((psync == 0).all())                        # pSync back at SYNC_VALUE
        rt.barrier_all()
        assert me % 2 == 0 or bool((dst == 0).all())
    run_threads(4, body, heap_bytes=1 << 20)


def test_teams_split_translate_reuse_and_limit():
    def body(rt):
        me, n = rt.my_pe, rt.n_pes
        w = rt.team_world
        even = rt.team_split_strided(w, 0, 2, 2)                   # {0, 2}
        if me in (0, 2):
            assert even.valid and even.n_pes == 2 and even.my_pe == me // 2
            assert even.translate_pe(1, w) == 2 and w.translate_pe(2, even) == 1 and w.translate_pe(1, even) == -1
        else:
            assert not even.valid and even.n_pes == -1 and even.my_pe == -1
        with pytest.raises(shmem.ShmemError):
            rt.team_split_strided(w, 0, 3, 3)                      # would run past the parent
        with pytest.raises(shmem.ShmemError):
            rt.team_split_strided(w, 5, 1, 1)
        # team collectives, back to back (shmem_team_b2b_collectives)
        if even.valid:
            s = rt.empty((10,), torch.float32, collective=False)
            d = rt.empty((10,), torch.float32, collective=False)
        else:
            s = rt.empty((10,), torch.float32, collective=False)
            d = rt.empty((10,), torch.float32, collective=False)
        s.fill_(me + 1.0)
        rt.barrier_all()
        if even.valid:
            for _ in range(20):
                rt.reduce(d, s, "sum", team=even)
                assert bool((d == 4.0).all())
            sub = rt.team_split_strided(even, 1, 1, 1)             # {2} as a team of the team
            if me == 2:
                assert sub.valid and sub.n_pes == 1 and sub.translate_pe(0, w) == 2
                sub.destroy()
            even.destroy()
        rt.barrier_all()
        # slots are recycled: 39 user teams can be live at once, the 40th split reports the limit
        teams = []
        for _ in range(39):
            teams.append(rt.team_split_strided(w, 0, 1, n))
        assert all(t.valid for t in teams) and len({t.slot for t in teams}) == 39
        with pytest.raises(shmem.ShmemError):
            rt.team_split_strided(w, 0, 1, n)
        for t in teams:
            t.destroy()
        again = rt.team_split_strided(w, 0, 1, n)
        assert again.valid
        again.sync()
        again.destroy()
        rt.team_world.destroy()                                    # no-op
        rt.barrier_all()
    run_threads(4, body, heap_bytes=1 << 20, timeout_s=120)


def test_contexts_many_and_team_relative():
    def body(rt):
        me, n = rt.my_pe, rt.n_pes
        ctxs = [rt.ctx_create(shmem.CTX_WG_PRIVATE if i % 2 else 0) for i in range(32)]   # many-ctx
        assert len({c.idx for c in ctxs}) == 32 and all(c.idx > 0 for c in ctxs)
        sym = rt.zeros((32,), torch.int32)
        for i, c in enumerate(ctxs):
            c.put(sym[i:i + 1], torch.tensor([me + 1], dtype=torch.int32), (me + 1) % n)
            c.quiet()
        rt.barrier_all()
        assert bool((sym == (me - 1) % n + 1).all())
        more = [rt.ctx_create() for _ in range(7)]                 # 39 user contexts in total
        with pytest.raises(shmem.ShmemError):
            rt.ctx_create()
        for c in ctxs + more:
            c.destroy()
        odd = rt.team_split_strided(None, 1, 2, 2)                 # {1, 3}
        if odd.valid:
            with rt.ctx_create(0, odd) as c:                       # PE numbers are team-relative
                c.put(sym[:1], torch.tensor([100 + me], dtype=torch.int32), 1 - odd.my_pe)
            odd.sync()
            assert int(sym[0]) == 100 + (3 if me == 1 else 1)
            odd.destroy()
        rt.barrier_all()
        st = rt.stats()
        assert st["ctx_create"] >= 39 and st["put"] >= 32 and st["team_split"] >= 1
    run_threads(4, body, heap_bytes=1 << 20)


def test_private_context_is_refused_from_another_thread_in_debug_mode():
    """CTX_PRIVATE promises use by the creating thread only; with debug checks on, another thread's call is refused
    (without them it is the caller's responsibility, as in the specification)."""
    import threading

    def body(rt):
        sym = rt.zeros((4,), torch.int32)
        priv = rt.ctx_create(shmem.CTX_WG_PRIVATE)
        ser = rt.ctx_create(shmem.CTX_SERIALIZED)
        one = torch.tensor([7], dtype=torch.int32)
        priv.put(sym[:1], one, rt.my_pe)                       # the creator may use it
        seen = {}

        def other():
            try:
                priv.put(sym[1:2], one, rt.my_pe)
                seen["priv"] = "accepted"
            except shmem.ShmemError as e:
                seen["priv"] = "refused"
            ser.put(sym[2:3], one, rt.my_pe)                   # SERIALIZED: any one thread at a time
            ser.quiet()
            seen["ser"] = "accepted"
        t = threading.Thread(target=other)
        t.start()
        t.join()
        priv.quiet()
        assert seen == {"priv": "refused", "ser": "accepted"}
        assert sym.tolist() == [7, 0, 7, 0]
        priv.destroy()
        ser.destroy()
    run_threads(1, body, config=Config.from_env(backend="cpu", heap_bytes=1 << 20, debug=True))


def test_malloc_semantics():
    def body(rt):
        assert rt.malloc(0) == 0                                   # malloc(0) -> null (collective)
        a = rt.malloc(100)
        b = rt.malloc(100)
        assert a and b and b - a == 128                            # rounded to 128-byte blocks
        rt.free_ptr(a)
        rt.free_ptr(b)
        u = rt.heap_usage()
        assert u["live_blocks"] == 0
        with pytest.raises(shmem.ShmemError):
            rt.empty((1 << 30,), torch.float32)                    # exhaustion is an error, not an abort
        rt.barrier_all()
        return a
    res = run_threads(2, body, heap_bytes=1 << 20)
    assert res[0] != res[1]                                        # heaps sit at different addresses...
    # ...but at identical offsets (checked by the symmetric put tests)


def test_pi_monte_carlo_and_circular_shift():
    def body(rt):
        me, n = rt.my_pe, rt.n_pes
        g = torch.Generator().manual_seed(me)
        pts = torch.rand(20000, 2, generator=g)
        inside = rt.empty((1,), torch.int64)
        total = rt.empty((1,), torch.int64)
        inside[0] = int(((pts ** 2).sum(1) <= 1).sum())
        rt.reduce(total, inside, "sum")
        pi = 4.0 * int(total[0]) / (20000 * n)
        assert abs(pi - math.pi) < 0.05
        a = rt.empty((1,), torch.int32)
        rt.put(a, torch.tensor([me], dtype=torch.int32), (me + 1) % n)     # source on the "stack"
        rt.barrier_all()
        assert int(a[0]) == (me - 1) % n
    run_threads(4, body, heap_bytes=1 << 20)


def test_typed_c_api_through_ctypes():
    """The handle-free typed names act on the calling thread's current PE."""
    def body(rt):
        lib = rt.lib
        me, n = rt.my_pe, rt.n_pes
        lib.bshmem_long_atomic_fetch_add.restype = C.c_long
        lib.bshmem_long_atomic_fetch_add.argtypes = [C.c_void_p, C.c_long, C.c_int]
        lib.bshmem_int_put.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int]
        lib.bshmem_double_g.restype = C.c_double
        lib.bshmem_double_g.argtypes = [C.c_void_p, C.c_int]
        lib.bshmem_double_p.argtypes = [C.c_void_p, C.c_double, C.c_int]
        lib.bshmem_float_sum_reduce.argtypes = [C.c_int32, C.c_void_p, C.c_void_p, C.c_size_t]
        lib.bshmem_int_wait_until.argtypes = [C.c_void_p, C.c_int, C.c_int]
        ctr = rt.zeros((1,), torch.int64)
        ints = rt.zeros((8,), torch.int32)
        dbl = rt.zeros((1,), torch.float64)
        fl = rt.empty((16,), torch.float32)
        fo = rt.empty((16,), torch.float32)
        lib.bshmem_long_atomic_fetch_add(ctr.data_ptr(), 2, 0)
        src = (C.c_int * 8)(*[me * 10 + i for i in range(8)])
        assert lib.bshmem_int_put(ints.data_ptr(), C.addressof(src), 8, (me + 1) % n) == 0
        lib.bshmem_double_p(dbl.data_ptr(), 1.25 + me, (me + 1) % n)
        rt.barrier_all()
        assert ints.tolist() == [((me - 1) % n) * 10 + i for i in range(8)]
        assert lib.bshmem_double_g(dbl.data_ptr(), me) == 1.25 + (me - 1) % n
        if me == 0:
            assert int(ctr[0]) == 2 * n
        fl.fill_(1.0)
        assert lib.bshmem_float_sum_reduce(0, fo.data_ptr(), fl.data_ptr(), 16) == 0
        assert bool((fo == float(n)).all())
        assert lib.bshmem_int_wait_until(ints.data_ptr(), 3, ((me - 1) % n) * 10) == 0       # GE
        rt.barrier_all()
        # typed put-with-signal (OpenSHMEM 1.5 names): the neighbour sees the data once its signal word counts 1
        lib.bshmem_float_put_signal.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_uint64, C.c_int, C.c_int]
        lib.bshmem_ctx_float_put_signal_nbi.argtypes = [C.c_int32] + lib.bshmem_float_put_signal.argtypes
        lib.bshmem_uint64_wait_until.argtypes = [C.c_void_p, C.c_int, C.c_uint64]
        sig = rt.zeros((2,), torch.int64)
        vals = (C.c_float * 16)(*[me + 0.5] * 16)
        assert lib.bshmem_float_put_signal(fo.data_ptr(), C.addressof(vals), 16, sig.data_ptr(), 1, 1, (me + 1) % n) == 0
        assert lib.bshmem_uint64_wait_until(sig.data_ptr(), 3, 1) == 0                      # GE 1
        assert bool((fo == (me - 1) % n + 0.5).all())
        assert lib.bshmem_ctx_float_put_signal_nbi(0, fl.data_ptr(), C.addressof(vals), 16, sig[1:].data_ptr(), 7, 0,
                                                   (me + 1) % n) == 0
        assert lib.bshmem_uint64_wait_until(sig[1:].data_ptr(), 0, 7) == 0                  # EQ 7
        assert bool((fl == (me - 1) % n + 0.5).all())
        rt.barrier_all()
    run_threads(2, body, heap_bytes=1 << 20)


def test_failure_detection_timeouts_dead_marks_and_global_exit():
    def body(rt):
        me = rt.my_pe
        flag = rt.zeros((1,), torch.int64)
        rt.barrier_all()
        if me == 0:
            with temporary_timeout(rt, 100):
                with pytest.raises(shmem.ShmemTimeout):
                    rt.wait_until(flag, "eq", 1)                   # nobody sets it
            rec = rt.error_record()
            assert rec["code"] == 3 and rec["where"] == 1
            assert rt.stats()["timeouts"] >= 1
            with temporary_timeout(rt, 200):
                with pytest.raises(shmem.ShmemTimeout):
                    rt.barrier_all()                               # PE 1 never joins this one
            rec = rt.error_record()
            assert rec["where"] == 2 and rec["pe"] == 1
        return True
    assert all(run_threads(2, body, heap_bytes=1 << 20))

    # a peer marked dead by the host ends the wait at once with ShmemAborted
    from roc_shmem_b200.cpu import CpuWorld
    world = CpuWorld(2, 1 << 20)
    rt0 = world.attach(0, Config.from_env(backend="cpu", heap_bytes=1 << 20, timeout_ms=20000))
    world.mark_dead(1)
    with pytest.raises(shmem.ShmemAborted):
        rt0.barrier_all()
    rt0.global_exit(3)                                             # raises the job-wide abort flag
    rt1 = world.attach(1, Config.from_env(backend="cpu", heap_bytes=1 << 20, timeout_ms=20000))
    with pytest.raises(shmem.ShmemAborted):
        rt1.barrier_all()
    rt0.finalize(); rt1.finalize(); world.close()


def test_finalize_then_init_again():
    for _ in range(2):
        assert run_threads(2, lambda rt: rt.barrier_all() or rt.my_pe, heap_bytes=1 << 20) == [0, 1]
