"""Host threads on the NVLink backend (clients/sos_tests: mt_contention.c, mt_a2a.c, threading.c, many-ctx.cpp,
put_ctx_mbw_mr.cpp): eight threads share the default context, every thread owns a context of its own, and a
context is an ordering domain — completing one context's operations does not wait for another's."""
import threading
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def _in_threads(n, fn):
    errs = []

    def wrap(t):
        try:
            torch.cuda.set_device(0)
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


def test_eight_threads_share_the_default_context_and_own_contexts():
    import roc_shmem_b200 as shmem
    rt = shmem.init("device", rank=0, world_size=1, heap_bytes=256 << 20, timeout_ms=5000)
    try:
        assert rt.query_thread() == shmem.THREAD_MULTIPLE
        NT, ITERS, WINDOW = 8, 50, 64
        ctr = rt.zeros((2,), torch.int64)
        fetched = [[] for _ in range(NT)]

        def contend(t):
            for _ in range(ITERS):
                fetched[t].append(rt.atomic_fetch_add(ctr, 1, 0))      # every thread reads ITS OWN answer
                rt.atomic_add(ctr[1:], 2, 0)
        _in_threads(NT, contend)
        rt.quiet()
        assert ctr.tolist() == [NT * ITERS, 2 * NT * ITERS]
        allv = sorted(v for f in fetched for v in f)
        assert allv == list(range(NT * ITERS))                         # no answer lost, none seen twice

        # many-ctx / put_ctx_mbw_mr: one context per thread, windows of non-blocking puts closed by the context's quiet
        sym = rt.zeros((NT * WINDOW,), torch.int32)
        srcs = [torch.zeros(WINDOW, dtype=torch.int32, device=rt.device) for _ in range(NT)]

        def windows(t):
            with rt.ctx_create(shmem.CTX_WG_PRIVATE if t % 2 else shmem.CTX_SERIALIZED) as c:
                for loop in range(4):
                    srcs[t].copy_(torch.arange(WINDOW, dtype=torch.int32, device=rt.device) + 1000 * loop + 10 * t)
                    torch.cuda.current_stream().synchronize()
                    for i in range(WINDOW):
                        c.put(sym[t * WINDOW + i:t * WINDOW + i + 1], srcs[t][i:i + 1], 0, nbi=True)
                    c.quiet()
        _in_threads(NT, windows)
        exp = torch.stack([torch.arange(WINDOW, dtype=torch.int32) + 3000 + 10 * t for t in range(NT)]).to(rt.device)
        assert torch.equal(sym.view(NT, WINDOW), exp)
        assert rt.stats()["ctx_create"] >= NT
    finally:
        shmem.finalize()


def test_a_context_is_its_own_ordering_domain():
    """Context A has a wait pending on its stream; context B's fetching atomic (which completes B's stream) must
    return at once, and B then releases A.  On a shared stream B would sit behind A until A's bounded wait ran out."""
    import roc_shmem_b200 as shmem
    rt = shmem.init("device", rank=0, world_size=1, heap_bytes=256 << 20, timeout_ms=8000)
    try:
        flag = rt.zeros((2,), torch.int64)
        a, b = rt.ctx_create(), rt.ctx_create()
        done = []

        def waiter(_):
            rt.bind_thread(a)                            # this thread's calls run on A's stream
            rt.wait_until(flag, "eq", 1)                 # spins on the device (bounded by the runtime's time limit)
            done.append(time.time())
            rt.bind_thread(None)
        th = threading.Thread(target=lambda: _in_threads(1, waiter))
        th.start()
        time.sleep(0.3)
        assert not done                                  # A is still waiting
        t0 = time.time()
        assert b.atomic_fetch_add(flag[1:], 5, 0) == 0   # B's stream: not behind A's pending wait
        assert time.time() - t0 < 3.0
        b.atomic_set(flag, 1, 0)                          # releases A
        th.join(30)
        assert done and done[0] - t0 < 5.0
        a.quiet()
        assert rt.error_record()["code"] == 0            # A's wait ended because of the flag, not its time limit
        a.destroy()
        b.destroy()
    finally:
        shmem.finalize()
