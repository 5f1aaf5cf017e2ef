"""roc_shmem_b200 — a Blackwell-native, GPU-centric OpenSHMEM-style runtime.

Capabilities follow ROCm/ROC_SHMEM (library/include/roc_shmem.hpp): a symmetric
heap, host- and device-initiated put/get/atomics/wait/fence/quiet, contexts and
teams, barrier/broadcast/reduce/fcollect/alltoall and a reverse-offload proxy
mode — re-designed for one NVSwitch node of B200s: a CUDA-VMM heap mapped into
every peer over NVLink 5, device communication as plain peer loads/stores/atomics
from hand-written sm_100a kernels, a ``torch.distributed`` store bootstrap, and
fused tcgen05 GEMM + collective kernels on top.

Typical use (one process per GPU, launched by ``torchrun``)::

    import roc_shmem_b200 as shmem
    rt = shmem.init()                       # NVLink backend on a GPU box, CPU backend otherwise
    x = rt.empty((1 << 20,), torch.float32)  # symmetric tensor
    rt.put(x, local, pe=(rt.my_pe + 1) % rt.n_pes)
    rt.barrier_all()
    shmem.finalize()
"""
from __future__ import annotations

import os
import threading
import uuid
from typing import Optional

import torch

from .config import Config
from .runtime import (CTX_DEFAULT, CTX_NOSTORE, CTX_SERIALIZED, CTX_SHARED, CTX_WG_PRIVATE, TEAM_INVALID, TEAM_WORLD,
                      Context, Runtime, Team)
from .utils.errors import ShmemAborted, ShmemError, ShmemTimeout

__version__ = "0.1.0"

_default: Optional[Runtime] = None
_tls = threading.local()


def current() -> Runtime:
    """The calling thread's PE (thread PEs) or the process-wide one."""
    rt = getattr(_tls, "rt", None) or _default
    if rt is None:
        raise ShmemError(5, "roc_shmem_b200.init() has not been called")
    return rt


def set_current(rt: Optional[Runtime]) -> None:
    _tls.rt = rt
    if rt is not None:
        rt.make_current()


def init(backend: Optional[str] = None, *, rank: Optional[int] = None, world_size: Optional[int] = None, store=None,
         device: Optional[int] = None, **config) -> Runtime:
    """Create this process's PE.  `backend`: "device" (NVLink), "proxy" (device
    API through the reverse-offload ring), "cpu", or None/"auto"."""
    global _default
    cfg = Config.from_env(backend=backend, **config)
    be = cfg.backend
    if be == "auto":
        be = "device" if torch.cuda.is_available() else "cpu"
    from .bootstrap import Bootstrap
    boot = Bootstrap.from_env(rank, world_size, store)
    if be == "cpu":
        from .cpu import CpuWorld
        if boot.world_size == 1:
            world = CpuWorld(1, cfg.heap_bytes)
        else:
            name = boot.broadcast(f"/bshmem-{uuid.uuid4().hex[:16]}" if boot.rank == 0 else None)
            if boot.rank == 0:
                world = CpuWorld(boot.world_size, cfg.heap_bytes, name=name, create=True)
            boot.barrier("cpu-world-created")
            if boot.rank != 0:
                world = CpuWorld(boot.world_size, cfg.heap_bytes, name=name, create=False)
        rt = world.attach(boot.rank, cfg)
        rt.bootstrap = boot
        boot.barrier("cpu-attached")
    else:
        from .gpu import init_device_runtime
        rt = init_device_runtime(boot, cfg, device=device, proxy=(be == "proxy"))
    _default = rt
    rt.make_current()
    return rt


def finalize() -> None:
    global _default
    rt = _default
    if rt is None:
        return
    boot = getattr(rt, "bootstrap", None)
    try:
        if boot is not None and boot.world_size > 1:
            boot.barrier("finalize")
    finally:
        rt.finalize()
        world = getattr(rt, "world", None)
        if world is not None and hasattr(world, "close"):
            world.close()
        _default = None


def global_exit(status: int = 0) -> None:
    """Abort the whole job: peers blocked in a wait get ShmemAborted; this process exits."""
    rt = current()
    rt.global_exit(status)
    os._exit(status)


# handle-free conveniences mirroring the OpenSHMEM names ---------------------------------
def my_pe() -> int: return current().my_pe
def n_pes() -> int: return current().n_pes
def barrier_all() -> None: current().barrier_all()
def sync_all() -> None: current().sync_all()
def empty(shape, dtype=torch.float32, **kw): return current().empty(shape, dtype, **kw)
def zeros(shape, dtype=torch.float32, **kw): return current().zeros(shape, dtype, **kw)
def free(t) -> None: current().free(t)
def put(dest, src, pe, **kw) -> None: current().put(dest, src, pe, **kw)
def get(dest, src, pe, **kw) -> None: current().get(dest, src, pe, **kw)
def fence() -> None: current().fence()
def quiet() -> None: current().quiet()


__all__ = ["init", "finalize", "global_exit", "current", "set_current", "Config", "Runtime", "Team", "Context",
           "ShmemError", "ShmemTimeout", "ShmemAborted", "TEAM_WORLD", "TEAM_INVALID", "CTX_DEFAULT", "CTX_NOSTORE",
           "CTX_SERIALIZED", "CTX_WG_PRIVATE", "CTX_SHARED", "my_pe", "n_pes", "barrier_all", "sync_all", "empty",
           "zeros", "free", "put", "get", "fence", "quiet", "init_thread", "THREAD_SINGLE", "THREAD_FUNNELED",
           "THREAD_WG_FUNNELED", "THREAD_SERIALIZED", "THREAD_MULTIPLE"]


# thread levels, values of bshmem_thread_level_t (csrc/include/bshmem_types.h)
THREAD_SINGLE, THREAD_FUNNELED, THREAD_WG_FUNNELED, THREAD_SERIALIZED, THREAD_MULTIPLE = 0, 1, 2, 3, 4


def init_thread(requested: int = THREAD_MULTIPLE, backend: Optional[str] = None, **kw):
    """`init` plus the thread-level handshake of roc_shmem_init_thread (library/include/roc_shmem.hpp:160-170):
    returns (runtime, provided).  Every backend here provides THREAD_MULTIPLE whatever is requested."""
    rt = init(backend, **kw)
    return rt, rt.query_thread()
