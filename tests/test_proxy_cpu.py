"""Reverse-offload ring + service thread on the CPU backend, with host producers: every
command type gives the same result as the direct call, and injected host-side faults
(paused service thread, dropped descriptor) surface as bounded-wait timeouts."""
import threading

import pytest
import torch

import roc_shmem_b200 as shmem
from roc_shmem_b200.cpu import run_threads
from roc_shmem_b200.proxy import Proxy
from roc_shmem_b200.utils import dtypes as D


def test_proxy_executes_every_command_type():
    def body(rt):
        me, n = rt.my_pe, rt.n_pes
        px = Proxy(rt, capacity=64, timeout_ms=10000)
        try:
            buf = rt.zeros((512,), torch.int64)
            src = torch.arange(512, dtype=torch.int64) + 1000 * me
            px.put(buf, src, (me + 1) % n)
            px.barrier_all()
            assert torch.equal(buf, torch.arange(512, dtype=torch.int64) + 1000 * ((me - 1) % n))
            got = torch.zeros(512, dtype=torch.int64)
            px.get(got, buf, (me + 1) % n)
            assert torch.equal(got, src)
            sym_src = rt.empty((512,), torch.int64)
            sym_src.copy_(src)
            px.put(buf, sym_src, me, nbi=True)                 # symmetric source goes as a heap offset
            px.quiet()
            assert torch.equal(buf, src)
            px.barrier_all()
            px.p(buf, 77, (me + 1) % n)
            px.fence()
            px.sync_all()
            assert px.g(buf, me) == 77
            ctr = rt.zeros((1,), torch.int64)
            old = [px.amo(D.AMO_FETCH_ADD, ctr, 1, 0, 0) for _ in range(20)]
            px.barrier_all()
            assert px.g(ctr, 0) == 20 * n and len(set(old)) == 20
            px.barrier_all()                                   # everyone has read the total before it is swapped
            assert px.amo(D.AMO_FETCH_CSWAP, ctr, 5, 20 * n, 0) in (20 * n, 5)
            px.barrier_all()
            sig = rt.zeros((1,), torch.int64)
            px.put_signal(buf, src, sig, 9, (me + 1) % n)
            rt.wait_until(sig, "eq", 9)
            assert torch.equal(buf, torch.arange(512, dtype=torch.int64) + 1000 * ((me - 1) % n))
            px.barrier_all()
            red = rt.empty((512,), torch.int64)
            px.to_all(red, sym_src, "sum")
            assert torch.equal(red, sum(torch.arange(512, dtype=torch.int64) + 1000 * p for p in range(n)))
            bc = rt.zeros((512,), torch.int64)
            px.broadcast(bc, sym_src, 0)
            assert me == 0 or torch.equal(bc, torch.arange(512, dtype=torch.int64))
            fc = rt.empty((512 * n,), torch.int64)
            px.fcollect(fc, sym_src)
            assert fc.view(n, 512)[:, 0].tolist() == [1000 * p for p in range(n)]
            a2a = rt.empty((512 * n,), torch.int64)
            px.alltoall(a2a, fc)
            assert a2a.view(n, 512)[:, 0].tolist() == [1000 * me] * n
            c = px.counters()
            assert c["processed"] >= 30 and c["rma"] > 0 and c["amo"] >= 20 and c["coll"] > 0 and c["order"] >= 2
            assert c["errors"] == 0 and c["dropped"] == 0
            rt.barrier_all()
        finally:
            px.stop()
    run_threads(2, body, heap_bytes=4 << 20)


def test_many_host_producers_share_one_ring():
    def body(rt):
        px = Proxy(rt, capacity=8, timeout_ms=10000)          # small ring: back-pressure is exercised
        ctr = rt.zeros((1,), torch.int64)
        def worker():
            for _ in range(200):
                px.amo(D.AMO_ADD, ctr, 1, 0, 0)
        ts = [threading.Thread(target=worker) for _ in range(4)]
        [t.start() for t in ts]
        [t.join() for t in ts]
        px.quiet()
        rt.barrier_all()
        if rt.my_pe == 0:
            assert int(ctr[0]) == 800 * rt.n_pes
        rt.barrier_all()
        px.stop()
    run_threads(2, body, heap_bytes=1 << 20)


def test_paused_proxy_times_out_then_recovers():
    def body(rt):
        px = Proxy(rt, capacity=16, timeout_ms=150)
        x = rt.zeros((4,), torch.int32)
        ones = torch.ones(4, dtype=torch.int32)               # stays alive: the command runs later
        px.pause(True)
        with pytest.raises(shmem.ShmemTimeout):
            px.put(x, ones, 0)                                # nobody services the ring
        px.pause(False)
        px.set_timeout_ms(10000)
        px.quiet()                                            # the stalled put executes once the thread resumes
        assert x.tolist() == [1, 1, 1, 1]
        px.stop()
    run_threads(1, body, heap_bytes=1 << 20)


def test_dropped_descriptor_times_out_only_that_command():
    def body(rt):
        px = Proxy(rt, capacity=16, timeout_ms=150)
        x = rt.zeros((4,), torch.int32)
        px.drop_next(1)
        with pytest.raises(shmem.ShmemTimeout):
            px.put(x, torch.full((4,), 5, dtype=torch.int32), 0)
        assert x.tolist() == [0, 0, 0, 0]                     # the dropped command never ran
        px.put(x, torch.full((4,), 6, dtype=torch.int32), 0)  # the next one does
        assert x.tolist() == [6, 6, 6, 6]
        assert px.counters()["dropped"] == 1
        px.stop()
    run_threads(1, body, heap_bytes=1 << 20)


def test_full_ring_gives_up_without_leaving_a_hole():
    """A producer that times out on a FULL ring must not have taken a ticket: the consumer runs strictly in ticket
    order and would otherwise wait for ever for a slot nobody fills.  Pause the service thread, fill the ring with
    non-blocking commands, let further submissions time out, resume: everything queued and everything later runs."""
    def body(rt):
        px = Proxy(rt, capacity=4, timeout_ms=100)
        ctr = rt.zeros((1,), torch.int64)
        px.pause(True)
        for _ in range(4):                                     # exactly fills the ring; nothing is consumed
            px.amo(D.AMO_ADD, ctr, 1, 0, 0, blocking=False)
        for _ in range(3):
            with pytest.raises(shmem.ShmemTimeout):
                px.amo(D.AMO_ADD, ctr, 100, 0, 0, blocking=False)   # no room: gives up, reserves nothing
        px.pause(False)
        px.set_timeout_ms(10000)
        for _ in range(10):                                    # later operations all complete, in order
            px.amo(D.AMO_ADD, ctr, 1, 0, 0)
        px.quiet()
        assert int(ctr[0]) == 14                               # the 3 abandoned submissions never ran
        c = px.counters()
        assert c["processed"] >= 15 and c["errors"] == 0
        px.stop()
    run_threads(1, body, heap_bytes=1 << 20)
