"""Out-of-band bootstrap over a ``torch.distributed`` key-value store.

The reference bootstraps over MPI: ``MPI_Init_thread`` in a singleton
(library/src/mpi_init_singleton.cpp), ``MPI_Allgather`` of heap bases, IPC
handles and keys (memory/remote_heap_info.hpp:89-92, ipc_policy.cpp:40,75) and
``MPI_Barrier``.  There is no MPI here; the same three primitives — rank/size,
blob all-gather, barrier — run over a TCPStore/FileStore, and POSIX file
descriptors of CUDA VMM allocations travel over a Unix-domain socket
(``SCM_RIGHTS``), which a store cannot carry.
"""
from __future__ import annotations

import os
import pickle
import socket
import time
from datetime import timedelta
from typing import Optional

import torch.distributed as dist


class Bootstrap:
    def __init__(self, store, rank: int, world_size: int, prefix: str = "bshmem", timeout_s: float = 120.0):
        self.store = dist.PrefixStore(prefix, store)
        self.rank = rank
        self.world_size = world_size
        self.timeout_s = timeout_s
        self._seq = 0
        try:
            self.store.set_timeout(timedelta(seconds=timeout_s))
        except Exception:
            pass

    # ---- construction ------------------------------------------------------
    @classmethod
    def from_env(cls, rank: Optional[int] = None, world_size: Optional[int] = None, store=None,
                 timeout_s: float = 120.0, prefix: str = "bshmem") -> "Bootstrap":
        """Rank/size from arguments, an initialised process group, or the
        torchrun environment (RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT)."""
        if store is None and dist.is_available() and dist.is_initialized():
            rank = dist.get_rank() if rank is None else rank
            world_size = dist.get_world_size() if world_size is None else world_size
            from torch.distributed import distributed_c10d as c10d
            store = c10d._get_default_store()
        if rank is None:
            rank = int(os.environ.get("RANK", "0"))
        if world_size is None:
            world_size = int(os.environ.get("WORLD_SIZE", "1"))
        if store is None:
            if world_size == 1:
                store = dist.HashStore()
            else:
                host = os.environ.get("MASTER_ADDR", "127.0.0.1")
                port = int(os.environ.get("MASTER_PORT", "29500"))
                agent = os.environ.get("TORCHELASTIC_USE_AGENT_STORE", "") == "True"
                store = dist.TCPStore(host, port, world_size, is_master=(rank == 0 and not agent),
                                      timeout=timedelta(seconds=timeout_s), wait_for_workers=False)
        return cls(store, rank, world_size, prefix=prefix, timeout_s=timeout_s)

    # ---- primitives ------------------------------------------------------------
    def _key(self, tag: str) -> str:
        self._seq += 1
        return f"{tag}/{self._seq}"

    def allgather(self, obj, tag: str = "ag") -> list:
        """All-gather of picklable objects; every rank must call in the same order."""
        key = self._key(tag)
        self.store.set(f"{key}/{self.rank}", pickle.dumps(obj))
        out = []
        for r in range(self.world_size):
            out.append(pickle.loads(self.store.get(f"{key}/{r}")))   # get() blocks until the key exists
        return out

    def broadcast(self, obj, root: int = 0, tag: str = "bc"):
        key = self._key(tag)
        if self.rank == root:
            self.store.set(key, pickle.dumps(obj))
            return obj
        return pickle.loads(self.store.get(key))

    def barrier(self, tag: str = "bar") -> None:
        key = self._key(tag)
        n = self.store.add(key, 1)
        deadline = time.time() + self.timeout_s
        while n < self.world_size:
            if time.time() > deadline:
                raise TimeoutError(f"bootstrap barrier {key}: {n}/{self.world_size} ranks arrived")
            time.sleep(0.001)
            n = self.store.add(key, 0)

    # ---- file-descriptor exchange ---------------------------------------------------
    def exchange_fds(self, my_fds: list[int], tag: str = "fd") -> list[list[int]]:
        """Every rank offers `my_fds`; returns, per rank, that rank's descriptors
        re-opened in this process (own entry = the originals).  Descriptors cannot
        go through a store, so each rank listens on an abstract Unix socket whose
        name it publishes, and peers connect to collect the descriptors."""
        name = f"\0bshmem-{os.getpid()}-{self.rank}-{self._seq}-{time.time_ns()}"
        srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        srv.bind(name)
        srv.listen(self.world_size)
        names = self.allgather(name, tag=tag + "-name")
        got: list[list[int]] = [[] for _ in range(self.world_size)]
        got[self.rank] = list(my_fds)
        # Deterministic order avoids deadlock: lower rank serves first.
        import threading

        def serve():
            for _ in range(self.world_size - 1):
                conn, _ = srv.accept()
                with conn:
                    socket.send_fds(conn, [b"fds"], list(my_fds))
                    conn.recv(1)   # wait until the peer has the descriptors

        th = threading.Thread(target=serve, daemon=True)
        th.start()
        for r in range(self.world_size):
            if r == self.rank:
                continue
            c = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
            c.settimeout(self.timeout_s)
            c.connect(names[r])
            _, fds, _, _ = socket.recv_fds(c, 16, max(len(my_fds), 1) + 8)
            got[r] = list(fds)
            c.send(b"k")
            c.close()
        th.join(self.timeout_s)
        srv.close()
        self.barrier(tag + "-done")
        return got


class ExitWatcher:
    """Job-wide abort over the bootstrap store: the counterpart of the reference's roc_shmem_global_exit, which calls
    MPI_Abort (library/src/roc_shmem.cpp).  `raise_exit(status)` publishes the status; a daemon thread in every other
    rank polls the key (non-blocking `check`, every `period_s`) and calls `on_exit(status)` — by default it prints one
    line and ends the process with that status, whatever its main thread is blocked in.  Store errors (the store's
    host has gone at shutdown) end the watcher silently."""

    KEY = "global-exit"

    def __init__(self, boot: "Bootstrap", on_exit=None, period_s: float = 0.2):
        import threading
        self.boot, self.period_s = boot, period_s
        self.on_exit = on_exit or self._default_exit
        self._stop = threading.Event()
        self._raised = False
        self.thread = threading.Thread(target=self._run, name="bshmem-exit-watcher", daemon=True)
        self.thread.start()

    def _default_exit(self, status: int) -> None:
        import sys
        print(f"[bshmem pe {self.boot.rank}] global_exit({status}) was called by another PE: leaving", file=sys.stderr, flush=True)
        os._exit(status & 0xFF)

    def _run(self) -> None:
        while not self._stop.wait(self.period_s):
            try:
                if self.boot.store.check([self.KEY]):
                    status = int(pickle.loads(self.boot.store.get(self.KEY)))
                    if not self._raised:
                        self.on_exit(status)
                    return
            except Exception:
                return

    def raise_exit(self, status: int) -> None:
        """Publish the job's exit status (first caller wins is not needed: every value ends the job)."""
        self._raised = True
        self.boot.store.set(self.KEY, pickle.dumps(int(status)))

    def stop(self) -> None:
        """Ends the watcher (joined, so no store call is in flight when the interpreter or the store goes away)."""
        import threading
        self._stop.set()
        if threading.current_thread() is not self.thread:
            self.thread.join(timeout=2.0)

