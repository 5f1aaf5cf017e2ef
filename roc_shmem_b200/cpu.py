"""CPU backend front-end: PEs as threads of one process or as processes that
share a POSIX shared-memory heap.

This is the fake the reference's test-suite lacks (it can only run as a real
MPI job on GPUs, clients/functional_tests/tester.cpp:494-564): everything except
NVLink data movement is testable without a GPU, and the GPU paths are compared
bitwise against it.
"""
from __future__ import annotations

import ctypes as C
import threading
import traceback
from typing import Callable, Optional, Sequence

import numpy as np
import torch

from . import _native
from .config import Config
from .runtime import Runtime
from .utils.errors import raise_for_status


def _cpu_tensor_from_ptr(ptr: int, shape, dtype) -> torch.Tensor:
    n = 1
    for s in shape:
        n *= s
    nbytes = max(n * torch.empty((), dtype=dtype).element_size(), 1)
    buf = (C.c_char * nbytes).from_address(ptr)
    t = torch.frombuffer(buf, dtype=dtype, count=n) if n else torch.empty(0, dtype=dtype)
    return t.view(*shape) if n else t.reshape(shape)


def native_config(cfg: Config) -> _native.NativeConfig:
    nc = _native.NativeConfig()
    _native.host_lib().bshmem_config_default(C.byref(nc))
    nc.heap_bytes = cfg.heap_bytes
    nc.timeout_us = cfg.timeout_ms * 1000
    nc.max_teams = cfg.max_teams
    nc.max_ctxs = cfg.max_ctxs
    nc.debug = int(cfg.debug)
    nc.profile = int(cfg.profile)
    return nc


class CpuWorld:
    """The shared mapping holding every PE's heap plus the control block."""

    def __init__(self, n_pes: int, heap_bytes: int, name: Optional[str] = None, create: bool = True):
        self.lib = _native.host_lib()
        self.n_pes = n_pes
        self.name = name
        w = C.c_void_p()
        if create:
            st = self.lib.bshmem_cpu_world_create(name.encode() if name else None, n_pes, heap_bytes, C.byref(w))
        else:
            st = self.lib.bshmem_cpu_world_open(name.encode(), C.byref(w))
        raise_for_status(st, f"cpu world {'create' if create else 'open'} failed")
        self.handle = w
        self._attached = 0
        self._lock = threading.Lock()
        self._closed = False

    def attach(self, pe: int, cfg: Optional[Config] = None) -> Runtime:
        cfg = cfg or Config.from_env(backend="cpu")
        nc = native_config(cfg)
        h = C.c_void_p()
        raise_for_status(self.lib.bshmem_cpu_init(self.handle, pe, C.byref(nc), C.byref(h)), "cpu init failed")
        with self._lock:
            self._attached += 1
        rt = Runtime(self.lib, h.value, tensor_from_ptr=_cpu_tensor_from_ptr, device=torch.device("cpu"),
                     on_finalize=self._detach)
        rt.backend = "cpu"
        rt.config = cfg
        rt.world = self
        return rt

    def _detach(self) -> None:
        with self._lock:
            self._attached -= 1

    def mark_dead(self, pe: int) -> None:
        """Host-side fault injection: peers waiting for `pe` get ShmemAborted."""
        raise_for_status(self.lib.bshmem_cpu_world_mark_dead(self.handle, pe))

    def close(self) -> None:
        if not self._closed:
            self._closed = True
            self.lib.bshmem_cpu_world_destroy(self.handle)


def run_threads(n_pes: int, fn: Callable[[Runtime], object], *, heap_bytes: int = 64 << 20,
                config: Optional[Config] = None, timeout_s: float = 120.0) -> list:
    """Run ``fn(rt)`` on `n_pes` PE threads over an anonymous shared heap and
    return the per-PE results; the first exception of any PE is re-raised."""
    cfg = config or Config.from_env(backend="cpu", heap_bytes=heap_bytes)
    world = CpuWorld(n_pes, cfg.heap_bytes)
    results: list = [None] * n_pes
    errors: list = [None] * n_pes

    def body(pe: int) -> None:
        rt = None
        try:
            rt = world.attach(pe, cfg)
            rt.make_current()
            results[pe] = fn(rt)
        except BaseException as e:  # noqa: BLE001 - reported to the caller below
            errors[pe] = (e, traceback.format_exc())
        finally:
            if rt is not None and not rt.finalized:
                try:
                    rt.finalize()
                except Exception:
                    pass

    threads = [threading.Thread(target=body, args=(pe,), name=f"bshmem-pe{pe}", daemon=True) for pe in range(n_pes)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout_s)
    hung = [t.name for t in threads if t.is_alive()]
    if hung:
        raise TimeoutError(f"PE threads still running after {timeout_s}s: {hung}")
    world.close()
    for pe, err in enumerate(errors):
        if err is not None:
            raise RuntimeError(f"PE {pe} failed:\n{err[1]}") from err[0]
    return results
