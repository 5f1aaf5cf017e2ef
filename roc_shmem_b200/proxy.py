"""Reverse-offload ("proxy") mode: operations travel as 128-byte descriptors through a
ring to a CPU service thread that executes them.

Parity: library/src/reverse_offload (ROBackend, Queue, MPITransport): the GPU enqueues
commands, a CPU thread runs them.  Here the same ring serves device producers (GPU
kernels, bshmem_proxy_device.cuh) and host producers (this module), every wait is
bounded, and the service thread has host-side fault-injection hooks (pause / drop).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from .utils import dtypes as D
from .utils.errors import raise_for_status

(OP_NOP, OP_PUT, OP_GET, OP_PUT_NBI, OP_GET_NBI, OP_P, OP_G, OP_AMO, OP_PUT_SIGNAL, OP_FENCE, OP_QUIET, OP_BARRIER_ALL,
 OP_SYNC_ALL, OP_TEAM_SYNC, OP_TO_ALL, OP_BROADCAST, OP_ALLTOALL, OP_FCOLLECT, OP_FINALIZE) = range(19)
FLAG_BLOCKING, FLAG_SRC_IS_OFFSET = 1, 2
COUNTER_NAMES = ("processed", "dropped", "idle_polls", "errors", "rma", "amo", "coll", "order")


class Desc(C.Structure):
    """Mirror of bshmem_proxy_desc_t."""
    _fields_ = [("op", C.c_uint32), ("pe", C.c_int32), ("dtype", C.c_uint32), ("sub_op", C.c_uint32),
                ("sym_off", C.c_uint64), ("local", C.c_uint64), ("nbytes", C.c_uint64), ("value", C.c_uint64),
                ("cond", C.c_uint64), ("flags", C.c_uint32), ("team", C.c_int32), ("root", C.c_uint32),
                ("block_id", C.c_uint32), ("ticket", C.c_uint64), ("pad", C.c_uint64 * 5), ("valid", C.c_uint64)]


assert C.sizeof(Desc) == 128


class Proxy:
    """Host handle of one PE's command ring + service thread."""

    def __init__(self, rt, capacity: int = 1024, timeout_ms: Optional[int] = None, handle: Optional[int] = None):
        self.rt = rt
        self.lib = rt.lib
        self._declare()
        if handle is None:
            px = C.c_void_p()
            tmo = (timeout_ms if timeout_ms is not None else rt.config.timeout_ms) * 1000
            raise_for_status(self.lib.bshmem_proxy_create_host(rt.h, capacity, tmo, C.byref(px)), "proxy create")
            self.px = px
        else:
            self.px = C.c_void_p(handle)
        self._base = int(self.lib.bshmem_heap_base(rt.h))
        self.stopped = False

    def _declare(self) -> None:
        lib = self.lib
        if getattr(lib, "_proxy_declared", False):
            return
        VP, I, U64 = C.c_void_p, C.c_int, C.c_uint64
        lib.bshmem_proxy_create_host.restype, lib.bshmem_proxy_create_host.argtypes = I, [VP, U64, U64, C.POINTER(VP)]
        lib.bshmem_proxy_host_submit.restype, lib.bshmem_proxy_host_submit.argtypes = I, [VP, C.POINTER(Desc), C.POINTER(U64)]
        lib.bshmem_proxy_pause.restype, lib.bshmem_proxy_pause.argtypes = I, [VP, I]
        lib.bshmem_proxy_drop_next.restype, lib.bshmem_proxy_drop_next.argtypes = I, [VP, I]
        lib.bshmem_proxy_get_counters.restype, lib.bshmem_proxy_get_counters.argtypes = I, [VP, C.POINTER(U64 * 8)]
        lib.bshmem_proxy_set_timeout_us.restype, lib.bshmem_proxy_set_timeout_us.argtypes = I, [VP, U64]
        lib.bshmem_proxy_stop.restype, lib.bshmem_proxy_stop.argtypes = I, [VP]
        lib._proxy_declared = True

    # ---- plumbing ---------------------------------------------------------------------
    def _off(self, t) -> int:
        return (t.data_ptr() if isinstance(t, torch.Tensor) else int(t)) - self._base

    def _local(self, t):
        """(value, flags) for a local buffer: heap offset if symmetric, raw pointer otherwise."""
        p = t.data_ptr() if isinstance(t, torch.Tensor) else int(t)
        if self.rt.is_symmetric(p):
            return p - self._base, FLAG_SRC_IS_OFFSET
        return p, 0

    def submit(self, d: Desc, blocking: bool = True) -> int:
        if blocking:
            d.flags |= FLAG_BLOCKING
        res = C.c_uint64(0)
        st = self.lib.bshmem_proxy_host_submit(self.px, C.byref(d), C.byref(res))
        raise_for_status(st, "proxy command")
        return res.value

    # ---- operations -----------------------------------------------------------------------
    def put(self, dest, src, pe: int, nbi: bool = False) -> None:
        loc, fl = self._local(src)
        d = Desc(op=OP_PUT_NBI if nbi else OP_PUT, pe=pe, sym_off=self._off(dest), local=loc,
                 nbytes=src.numel() * src.element_size(), flags=fl)
        self.submit(d, blocking=not nbi)

    def get(self, dest, src, pe: int, nbi: bool = False) -> None:
        loc, fl = self._local(dest)
        d = Desc(op=OP_GET_NBI if nbi else OP_GET, pe=pe, sym_off=self._off(src), local=loc,
                 nbytes=dest.numel() * dest.element_size(), flags=fl)
        self.submit(d, blocking=not nbi)

    def p(self, dest, value, pe: int) -> None:
        code = D.code_of(dest.dtype)
        self.submit(Desc(op=OP_P, pe=pe, dtype=code, sym_off=self._off(dest), value=D.to_bits(code, value)), blocking=False)

    def g(self, src, pe: int):
        code = D.code_of(src.dtype)
        return D.from_bits(code, self.submit(Desc(op=OP_G, pe=pe, dtype=code, sym_off=self._off(src))))

    def amo(self, op: int, dest, value=0, cond=0, pe: int = 0, blocking: bool = True):
        """One of the 15 atomics through the ring; a non-blocking submission returns nothing (use non-fetching ops)."""
        code = D.code_of(dest.dtype)
        r = self.submit(Desc(op=OP_AMO, pe=pe, dtype=code, sub_op=op, sym_off=self._off(dest), value=D.to_bits(code, value),
                             cond=D.to_bits(code, cond)), blocking=blocking)
        return D.from_bits(code, r) if blocking else None

    def put_signal(self, dest, src, sig, value: int, pe: int, sig_op: int = D.SIGNAL_SET) -> None:
        loc, fl = self._local(src)
        self.submit(Desc(op=OP_PUT_SIGNAL, pe=pe, sub_op=sig_op, sym_off=self._off(dest), local=loc,
                         nbytes=src.numel() * src.element_size(), value=value, cond=self._off(sig), flags=fl))

    def fence(self) -> None:
        self.submit(Desc(op=OP_FENCE))

    def quiet(self) -> None:
        self.submit(Desc(op=OP_QUIET))

    def barrier_all(self) -> None:
        self.submit(Desc(op=OP_BARRIER_ALL))

    def sync_all(self) -> None:
        self.submit(Desc(op=OP_SYNC_ALL))

    def to_all(self, dest, src, op="sum", team: int = 0) -> None:
        o = D.OPS[op] if isinstance(op, str) else int(op)
        self.submit(Desc(op=OP_TO_ALL, dtype=D.code_of(src.dtype), sub_op=o, sym_off=self._off(dest), local=self._off(src),
                         nbytes=src.numel(), team=team, flags=FLAG_SRC_IS_OFFSET))

    def broadcast(self, dest, src, root: int, team: int = 0) -> None:
        self.submit(Desc(op=OP_BROADCAST, sym_off=self._off(dest), local=self._off(src),
                         nbytes=src.numel() * src.element_size(), team=team, root=root, flags=FLAG_SRC_IS_OFFSET))

    def alltoall(self, dest, src, team: int = 0) -> None:
        n = self.rt.lib.bshmem_team_n_pes(self.rt.h, team)
        self.submit(Desc(op=OP_ALLTOALL, sym_off=self._off(dest), local=self._off(src),
                         nbytes=src.numel() * src.element_size() // n, team=team, flags=FLAG_SRC_IS_OFFSET))

    def fcollect(self, dest, src, team: int = 0) -> None:
        self.submit(Desc(op=OP_FCOLLECT, sym_off=self._off(dest), local=self._off(src),
                         nbytes=src.numel() * src.element_size(), team=team, flags=FLAG_SRC_IS_OFFSET))

    # ---- fault injection (host side only) and introspection ------------------------------------
    def pause(self, paused: bool = True) -> None:
        raise_for_status(self.lib.bshmem_proxy_pause(self.px, int(paused)))

    def drop_next(self, n: int = 1) -> None:
        raise_for_status(self.lib.bshmem_proxy_drop_next(self.px, n))

    def set_timeout_ms(self, ms: int) -> None:
        raise_for_status(self.lib.bshmem_proxy_set_timeout_us(self.px, ms * 1000))

    def counters(self) -> dict:
        arr = (C.c_uint64 * 8)()
        raise_for_status(self.lib.bshmem_proxy_get_counters(self.px, C.byref(arr)))
        return dict(zip(COUNTER_NAMES, (int(v) for v in arr)))

    def stop(self) -> None:
        if not self.stopped:
            self.stopped = True
            self.lib.bshmem_proxy_stop(self.px)


def attach_proxy(rt, capacity: Optional[int] = None) -> Proxy:
    """Create the PE's ring and service thread (GPU runtimes additionally get the device-side
    ring descriptor so kernels can enqueue commands)."""
    cap = capacity or rt.config.proxy_slots
    if getattr(rt, "backend", "cpu") == "cpu":
        rt.proxy = Proxy(rt, cap)
    else:
        from .gpu_proxy import attach_gpu_proxy
        rt.proxy = attach_gpu_proxy(rt, cap)
    return rt.proxy
