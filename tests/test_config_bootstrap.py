"""Config/env handling and the store bootstrap (rank/size, all-gather, barrier, fd passing)."""
import multiprocessing as mp
import os
import tempfile

import pytest
import torch.distributed as dist

from roc_shmem_b200.bootstrap import Bootstrap, ExitWatcher
from roc_shmem_b200.config import Config


def test_config_defaults_env_aliases_and_overrides(monkeypatch):
    c = Config.from_env()
    assert c.heap_bytes == 1 << 30 and c.max_teams == 40 and c.backend == "auto" and c.nvls == "auto"
    monkeypatch.setenv("ROC_SHMEM_HEAP_SIZE", "64M")           # the reference's spelling is accepted
    monkeypatch.setenv("B200SHMEM_MAX_NUM_TEAMS", "8")
    monkeypatch.setenv("B200SHMEM_DEBUG", "1")
    c = Config.from_env(timeout_ms=5)
    assert c.heap_bytes == 64 << 20 and c.max_teams == 8 and c.debug is True and c.timeout_ms == 5
    monkeypatch.setenv("B200SHMEM_HEAP_SIZE", "2GiB")          # the native spelling wins over the alias
    assert Config.from_env().heap_bytes == 2 << 30
    with pytest.raises(ValueError):
        Config.from_env(backend="mpi")
    with pytest.raises(ValueError):
        Config.from_env(proxy_slots=100)
    with pytest.raises(TypeError):
        Config.from_env(no_such_field=1)


def _boot_worker(rank, world, path, q):
    store = dist.FileStore(path, world)
    b = Bootstrap(store, rank, world, timeout_s=30)
    got = b.allgather({"rank": rank, "blob": bytes([rank]) * 3})
    b.barrier()
    root = b.broadcast("hello" if rank == 1 else None, root=1)
    r, w = os.pipe()
    os.write(w, f"from-{rank}".encode() * (world - 1))       # one 6-byte message per reader of this pipe
    fds = b.exchange_fds([r])
    texts = [os.read(fds[p][0], 6).decode() if p != rank else f"from-{rank}" for p in range(world)]
    q.put((rank, [g["rank"] for g in got], root, texts))


def test_bootstrap_allgather_barrier_broadcast_and_fd_exchange():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "store")
        procs = [ctx.Process(target=_boot_worker, args=(r, 3, path, q)) for r in range(3)]
        [p.start() for p in procs]
        res = sorted(q.get(timeout=120) for _ in range(3))
        [p.join(30) for p in procs]
    for rank, ranks, root, texts in res:
        assert ranks == [0, 1, 2] and root == "hello"
        assert texts == ["from-0", "from-1", "from-2"]        # each descriptor really is the peer's pipe


def test_bootstrap_with_eight_ranks():
    """The rank count of a full node: every rank serves its descriptor to seven peers while it collects theirs."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "store")
        procs = [ctx.Process(target=_boot_worker, args=(r, 8, path, q)) for r in range(8)]
        [p.start() for p in procs]
        res = sorted(q.get(timeout=180) for _ in range(8))
        [p.join(30) for p in procs]
    for rank, ranks, root, texts in res:
        assert ranks == list(range(8)) and root == "hello"
        assert texts == [f"from-{p}" for p in range(8)]


def test_bootstrap_barrier_times_out_when_a_rank_never_joins():
    b = Bootstrap(dist.HashStore(), 0, 2, timeout_s=0.3)
    with pytest.raises(TimeoutError):
        b.barrier()


def test_exit_watcher_delivers_the_status_to_every_other_rank():
    """global_exit over the store: the caller publishes a status; every other rank's watcher thread hands it to its
    exit hook (here a recorder instead of os._exit), and a stopped watcher stays silent."""
    import time
    store = dist.HashStore()
    ranks = [Bootstrap(store, r, 3, timeout_s=5) for r in range(3)]
    seen = {}
    watchers = [ExitWatcher(b, on_exit=lambda st, r=b.rank: seen.setdefault(r, st), period_s=0.01) for b in ranks]
    time.sleep(0.05)
    assert seen == {}
    watchers[2].stop()                       # rank 2 has finalised: it must not react any more
    time.sleep(0.05)
    watchers[1].raise_exit(42)
    deadline = time.time() + 5
    while 0 not in seen and time.time() < deadline:
        time.sleep(0.01)
    time.sleep(0.05)
    assert seen == {0: 42}                   # not the caller (it leaves by itself), not the stopped one
    for w in watchers:
        w.stop()


def _exit_worker(rank, world, path):
    import time
    b = Bootstrap(dist.FileStore(path, world), rank, world, timeout_s=30)
    w = ExitWatcher(b, period_s=0.02)
    b.barrier()
    if rank == 1:
        w.raise_exit(9)
        os._exit(9)
    time.sleep(30)                           # a blocked main thread: only the watcher can end this process
    os._exit(0)


def test_global_exit_ends_blocked_processes_with_the_status():
    ctx = mp.get_context("spawn")
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "store")
        procs = [ctx.Process(target=_exit_worker, args=(r, 3, path)) for r in range(3)]
        [p.start() for p in procs]
        [p.join(25) for p in procs]
        assert [p.exitcode for p in procs] == [9, 9, 9]
