"""More of the reference's host programs on the CPU backend (clients/sos_tests/): several threads per PE
(threading.c, thread_wait.c, mt_contention.c, mt_a2a.c), per-thread contexts under load (put_ctx_mbw_mr.cpp),
large transfers (bigput.c, bigget.c), broadcast flood (bcast_flood.c), max / big reductions
(max_reduction.c, big_reduction.c), the shmalloc size sweep (shmalloc.c), fetch-inc loop (lfinc.c) and
back-to-back team collectives (shmem_team_b2b_collectives.c)."""
import threading

import torch

import roc_shmem_b200 as shmem
from roc_shmem_b200.cpu import run_threads


def _in_threads(n, fn):
    """Run fn(tid) in n threads of the calling PE; re-raise the first failure."""
    errs = []

    def wrap(t):
        try:
            fn(t)
        except BaseException as e:  # noqa: BLE001
            errs.append(e)
    ths = [threading.Thread(target=wrap, args=(t,)) for t in range(n)]
    for t in ths:
        t.start()
    for t in ths:
        t.join(120)
    if errs:
        raise errs[0]


def test_mt_contention_atomics_from_eight_threads_per_pe():
    NT, ITERS = 8, 200

    def body(rt):
        me, n = rt.my_pe, rt.n_pes
        ctr = rt.zeros((1,), torch.int64)
        rt.barrier_all()
        _in_threads(NT, lambda t: [rt.atomic_add(ctr, 1, (me + 1) % n) for _ in range(ITERS)])
        rt.barrier_all()
        assert int(ctr[0]) == NT * ITERS
    run_threads(2, body, heap_bytes=1 << 20, timeout_s=180)


def test_mt_a2a_and_thread_wait():
    """Thread t of every PE puts to slot t of every other PE, then waits for its own slot's flags."""
    NT = 4

    def body(rt):
        me, n = rt.my_pe, rt.n_pes
        data = rt.zeros((NT * n,), torch.int64)
        flags = rt.zeros((NT * n,), torch.int64)
        rt.barrier_all()

        def work(t):
            for pe in range(n):
                rt.put(data[t * n + me:t * n + me + 1], torch.tensor([1000 * me + t], dtype=torch.int64), pe)
                rt.fence()
                rt.atomic_set(flags[t * n + me:t * n + me + 1], 1, pe)
            for src in range(n):
                rt.wait_until(flags[t * n + src:t * n + src + 1], "eq", 1)
                assert int(data[t * n + src]) == 1000 * src + t
        _in_threads(NT, work)
        rt.barrier_all()
    run_threads(3, body, heap_bytes=1 << 20, timeout_s=180)


def test_per_thread_contexts_message_rate_window():
    """put_ctx_mbw_mr: every thread owns a context, issues windows of 64 non-blocking puts and a quiet."""
    NT, WINDOW, LOOPS = 4, 64, 5

    def body(rt):
        me, n = rt.my_pe, rt.n_pes
        sym = rt.zeros((NT * WINDOW,), torch.int32)
        rt.barrier_all()

        def work(t):
            with rt.ctx_create(shmem.CTX_WG_PRIVATE if t % 2 else shmem.CTX_SERIALIZED) as c:
                src = torch.full((1,), 0, dtype=torch.int32)
                for loop in range(LOOPS):
                    for i in range(WINDOW):
                        src[0] = loop * 1000 + i
                        c.put(sym[t * WINDOW + i:t * WINDOW + i + 1], src, (me + 1) % n, nbi=False)
                    c.quiet()
        _in_threads(NT, work)
        rt.barrier_all()
        exp = torch.arange(WINDOW, dtype=torch.int32) + (LOOPS - 1) * 1000
        assert torch.equal(sym.view(NT, WINDOW), exp.expand(NT, WINDOW))
        assert rt.stats()["put"] >= NT * WINDOW * LOOPS
    run_threads(2, body, heap_bytes=1 << 20, timeout_s=180)


def test_bigput_bigget_and_shmalloc_sweep():
    def body(rt):
        me, n = rt.my_pe, rt.n_pes
        N = 1 << 21                                               # 16 MiB of int64
        big = rt.empty((N,), torch.int64)
        src = torch.arange(N, dtype=torch.int64) * (me + 1)
        rt.barrier_all()
        rt.put(big, src, (me + 1) % n)
        rt.barrier_all()
        assert torch.equal(big, torch.arange(N, dtype=torch.int64) * ((me - 1) % n + 1))
        got = torch.empty(N, dtype=torch.int64)
        rt.get(got, big, (me + 1) % n)
        assert torch.equal(got, src)
        rt.barrier_all()
        rt.free(big)
        # shmalloc sweep: powers of two up to 2^22 words, every block usable, everything returned
        for lg in range(0, 23, 3):
            t = rt.empty((1 << lg,), torch.int32)
            t.fill_(lg)
            assert int(t[-1]) == lg
            rt.free(t)
        assert rt.heap_usage()["live_blocks"] == 0
    run_threads(2, body, heap_bytes=64 << 20, timeout_s=180)


def test_bcast_flood_max_and_big_reduction_lfinc():
    def body(rt):
        me, n = rt.my_pe, rt.n_pes
        # bcast_flood: many back-to-back broadcasts of 100 KB, root rotating
        src = rt.empty((25600,), torch.int32)
        dst = rt.empty((25600,), torch.int32)
        for it in range(60):
            root = it % n
            src.fill_(it * 10 + me)
            dst.fill_(-1)
            rt.broadcast(dst, src, root)
            if me != root:
                assert int(dst[0]) == it * 10 + root and int(dst[-1]) == it * 10 + root
            else:
                assert int(dst[0]) == -1                           # the root's dest is untouched
        # max_reduction + big_reduction (1 Mi longs)
        a = rt.empty((1 << 20,), torch.int64)
        b = rt.empty((1 << 20,), torch.int64)
        a.copy_(torch.arange(1 << 20, dtype=torch.int64) + me)
        rt.reduce(b, a, "max")
        assert torch.equal(b, torch.arange(1 << 20, dtype=torch.int64) + n - 1)
        rt.reduce(b, a, "sum")
        assert torch.equal(b, torch.arange(1 << 20, dtype=torch.int64) * n + n * (n - 1) // 2)
        # lfinc: a long run of fetch-incs on PE 0 hands out every ticket exactly once
        ctr = rt.zeros((1,), torch.int64)
        rt.barrier_all()
        mine = [rt.atomic_fetch_inc(ctr, 0) for _ in range(500)]
        rt.barrier_all()
        tickets = rt.empty((500 * n,), torch.int64)
        mine_sym = rt.empty((500,), torch.int64)
        mine_sym.copy_(torch.tensor(mine, dtype=torch.int64))
        rt.fcollect(tickets, mine_sym)
        assert sorted(tickets.tolist()) == list(range(500 * n))
    run_threads(3, body, heap_bytes=64 << 20, timeout_s=240)


def test_team_back_to_back_collectives():
    def body(rt):
        me, n = rt.my_pe, rt.n_pes
        even = rt.team_split_strided(None, 0, 2, (n + 1) // 2)
        src = rt.empty((64,), torch.int32)
        dst = rt.empty((64 * n,), torch.int32)
        for it in range(40):                                        # no barrier between collectives of a team
            src.fill_(it + me)
            if even.valid:
                rt.reduce(dst[:64], src, "sum", team=even)
                members = list(range(0, n, 2))
                assert int(dst[0]) == sum(it + p for p in members)
                rt.broadcast(dst[:64], src, 0, team=even)
                rt.fcollect(dst[:64 * even.n_pes], src, team=even)
                assert [int(dst[64 * k]) for k in range(even.n_pes)] == [it + p for p in members]
            rt.reduce(dst[:64], src, "max")
            assert int(dst[0]) == it + n - 1
        if even.valid:
            even.destroy()
        rt.barrier_all()
    run_threads(4, body, heap_bytes=1 << 20, timeout_s=240)
