"""CPU backend across processes: PEs are separate processes sharing a POSIX shm heap, brought
up through shmem.init() with a TCP store (the same path torchrun-launched jobs take)."""
import multiprocessing as mp
import os
import socket

import torch


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import roc_shmem_b200 as shmem
    rt = shmem.init("cpu", heap_bytes=8 << 20, timeout_ms=20000)
    me, n = rt.my_pe, rt.n_pes
    x = rt.zeros((1000,), torch.int64)
    rt.put(x, torch.arange(1000) + 10000 * me, (me + 1) % n)
    rt.barrier_all()
    ok = bool(torch.equal(x, torch.arange(1000) + 10000 * ((me - 1) % n)))
    s = rt.empty((1000,), torch.int64)
    rt.reduce(s, x, "sum")
    ok &= bool(torch.equal(s, sum(torch.arange(1000) + 10000 * p for p in range(n))))
    c = rt.zeros((1,), torch.int64)
    for _ in range(100):
        rt.atomic_inc(c, 0)
    rt.barrier_all()
    ok &= rt.g(c, 0) == 100 * n
    team = rt.team_split_strided(None, 0, 1, 2)
    if team.valid:
        team.sync()
        team.destroy()
    rt.barrier_all()
    shmem.finalize()
    q.put((rank, ok))


def test_three_process_pes_over_posix_shm():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 3, port, q)) for r in range(3)]
    [p.start() for p in procs]
    res = sorted(q.get(timeout=180) for _ in range(3))
    [p.join(30) for p in procs]
    assert res == [(0, True), (1, True), (2, True)]
