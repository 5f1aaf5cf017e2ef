"""NVLink backend front-end: one process per GPU, heaps mapped into every peer.

Bring-up (the analogue of library/src/gpu_ib/backend_ib.cpp:70-111 and
ipc_policy.cpp:34-111, with the store bootstrap in place of MPI):

1. every PE creates its heap as a CUDA VMM allocation and exports a POSIX fd;
2. fds are exchanged over Unix sockets, every PE maps every peer's heap into one
   contiguous virtual range (``base + pe * heap_bytes``);
3. optionally the allocations are bound to an NVLink multicast object (NVLS);
4. the runtime handle is created on top of the mapped heap.

If the driver refuses shareable VMM allocations the heap falls back to
``cudaMalloc`` + ``cudaIpc`` handles, which travel through the store as bytes.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

from . import _native
from .bootstrap import Bootstrap
from .config import Config
from .cpu import native_config
from .runtime import Runtime
from .utils import dtypes as D
from .utils.errors import ShmemError, raise_for_status

_VP, _I, _U64 = C.c_void_p, C.c_int, C.c_uint64
_declared = False


class DevState(C.Structure):
    """Mirror of bshmem_dev_state_t (passed by value to user kernels)."""
    _fields_ = [("my_pe", C.c_int32), ("n_pes", C.c_int32), ("heap_bytes", C.c_uint64),
                ("heap_base", C.c_void_p * 16), ("mc_base", C.c_void_p), ("err", C.c_void_p),
                ("timeout_ns", C.c_ulonglong), ("stats", C.c_void_p), ("proxy", C.c_void_p),
                ("debug", C.c_uint32), ("reserved", C.c_uint32)]


DSTAT_NAMES = ("put", "get", "put_signal", "p", "g", "amo", "fence", "quiet", "wait", "wait_ns", "barrier",
               "barrier_ns", "coll", "bytes_put", "bytes_get", "timeouts", "proxy_ops")

TRACE_OPS = {1: "put", 2: "get", 3: "put_signal", 4: "amo", 5: "wait", 6: "barrier", 7: "coll", 8: "timeout"}

COLL_SYNC, COLL_BARRIER, COLL_BROADCAST, COLL_REDUCE, COLL_REDUCE_SCATTER, COLL_FCOLLECT, COLL_ALLTOALL = range(7)
COLL_REDUCE_ROOT = 8


def cuda_lib() -> C.CDLL:
    global _declared
    lib = _native.load("libbshmem_cuda.so")
    if not _declared:
        _native.declare_runtime_api(lib)

        def f(name, res, *args):
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, list(args)
        f("bshmem_gpu_last_error", C.c_char_p)
        f("bshmem_gpu_heap_create", _I, _I, _I, _U64, _I, _I, C.POINTER(_VP))
        f("bshmem_gpu_heap_create_local_group", _I, _I, _U64, _I, C.POINTER(_VP))
        f("bshmem_gpu_heap_export_fd", _I, _VP, C.POINTER(_I))
        f("bshmem_gpu_heap_import_fd", _I, _VP, _I, _I)
        f("bshmem_gpu_heap_export_ipc", _I, _VP, _VP)
        f("bshmem_gpu_heap_import_ipc", _I, _VP, _I, _VP)
        f("bshmem_gpu_multicast_supported", _I, _I)
        f("bshmem_gpu_multicast_create", _I, _VP, C.POINTER(_I))
        f("bshmem_gpu_multicast_import", _I, _VP, _I)
        f("bshmem_gpu_multicast_add_device", _I, _VP)
        f("bshmem_gpu_multicast_bind", _I, _VP)
        f("bshmem_gpu_heap_destroy", _I, _VP)
        f("bshmem_gpu_heap_bytes", _U64, _VP)
        f("bshmem_gpu_init", _I, _VP, C.POINTER(_native.NativeConfig), _I, _I, C.POINTER(_VP))
        f("bshmem_gpu_set_stream", _I, _VP, _VP)
        f("bshmem_gpu_set_blocking", _I, _VP, _I)
        f("bshmem_gpu_set_coll_ctas", _I, _VP, _I)
        f("bshmem_gpu_set_nvls", _I, _VP, _I)
        f("bshmem_gpu_get_state", _I, _VP, C.POINTER(DevState))
        f("bshmem_gpu_check_error", _I, _VP)
        f("bshmem_gpu_get_device_stats", _I, _VP, C.POINTER(_U64), _I)
        f("bshmem_gpu_reset_device_stats", _I, _VP)
        f("bshmem_gpu_trace_enable", _I, _VP, _I)
        f("bshmem_gpu_trace_read", _I, _VP, C.POINTER(_U64), _I, C.POINTER(_I), C.POINTER(_U64))
        f("bshmem_gpu_rma_kernel", _I, _VP, _VP, _VP, _U64, _I, _I, _I, _I, _I)
        f("bshmem_gpu_group_collective", _I, C.POINTER(_VP), _I, _I, _I, _I, _I, _I, _U64, _U64, _U64, _I)
        f("bshmem_gpu_group_team_split", _I, C.POINTER(_VP), _I, _I, _I, _I, _I, C.POINTER(_I))
        f("bshmem_gpu_get_stream", _I, _VP, C.POINTER(_VP))
        f("bshmem_gpu_synchronize", _I, _VP)
        f("bshmem_gpu_bench_pingpong", _I, _VP, _VP, _I, _I, _I, C.POINTER(_U64))
        f("bshmem_gpu_bench_put_signal", _I, _VP, _VP, _VP, _U64, _I, _I, _I, _I, C.POINTER(_U64))
        f("bshmem_gpu_bench_amo", _I, _VP, _VP, _I, _I, _I, C.POINTER(_U64))
        f("bshmem_gpu_bench_msgrate", _I, _VP, _VP, _VP, _U64, _I, _I, _I, _I, C.POINTER(_U64))
        f("bshmem_gpu_swarm_get", _I, _VP, _VP, _VP, _U64, _I, _I, _I)
        f("bshmem_gpu_api_selftest", _I, _VP, _VP, _VP, _VP, _I, _VP)
        f("bshmem_gpu_wg_collectives", _I, _VP, _VP, _VP, _I, C.POINTER(_I))
        f("bshmem_gpu_bench_amo_rate", _I, _VP, _VP, _I, _I, _I, _I, _I, C.POINTER(_U64))
        f("bshmem_gpu_put_signal_stream", _I, _VP, _VP, _VP, _VP, _U64, _I, _I, _I, _I)
        f("bshmem_gpu_api_matrix", _I, _VP, _VP, _I, _VP, _VP, _VP, _VP, _VP, _VP, _I, _I, _VP)
        f("bshmem_gpu_bind_thread_ctx", _I, _VP, _I)
        f("bshmem_gpu_functional_run", _I, _VP, _I, _I, _I, _I, _I, _I, _I, _U64, _VP, _VP, _VP, _VP, _VP, _VP, C.c_long, _I,
          C.c_uint, C.POINTER(C.c_float))
        f("bshmem_gpu_get_device", _I, _VP, C.POINTER(_I))
        _declared = True
    return lib


class _CudaArray:
    """Minimal __cuda_array_interface__ holder so torch can alias heap memory."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


def cuda_tensor_from_ptr(ptr: int, shape, dtype, device: torch.device) -> torch.Tensor:
    n = 1
    for s in shape:
        n *= s
    esz = torch.empty((), dtype=dtype).element_size()
    nbytes = max(n * esz, 1)
    raw = torch.as_tensor(_CudaArray(ptr, nbytes), device=device)
    if n == 0:
        return torch.empty(shape, dtype=dtype, device=device)
    return raw[: n * esz].view(dtype).view(*shape)


def _gpu_error(lib, what: str, status: int) -> None:
    if status != 0:
        msg = lib.bshmem_gpu_last_error()
        raise_for_status(status, f"{what}: {msg.decode() if msg else ''}")


class DeviceRuntime(Runtime):
    """Runtime over the NVLink backend, plus the GPU-only knobs."""

    backend = "device"

    def __init__(self, lib, handle, device: torch.device, heap, own_heap: bool = True):
        super().__init__(lib, handle,
                         tensor_from_ptr=lambda p, shape, dtype: cuda_tensor_from_ptr(p, shape, dtype, device),
                         device=device)
        self.heap = heap

    # stream-ordered mode: calls enqueue on `stream` and return; errors surface at quiet()
    def set_stream(self, stream: Optional[torch.cuda.Stream]) -> None:
        # None -> the runtime's own stream; a torch stream (the default stream included) is used as given
        s = C.c_void_p(stream.cuda_stream) if stream is not None else C.c_void_p(-1)
        self._check(self.lib.bshmem_gpu_set_stream(self.h, s))

    def set_blocking(self, blocking: bool) -> None:
        self._check(self.lib.bshmem_gpu_set_blocking(self.h, int(blocking)))

    def synchronize(self) -> None:
        """Host-side wait for everything enqueued on the PE's stream (stream mode's `quiet`)."""
        self._check(self.lib.bshmem_gpu_synchronize(self.h))

    def set_coll_ctas(self, n: int) -> None:
        self._check(self.lib.bshmem_gpu_set_coll_ctas(self.h, n))

    def set_nvls(self, on: bool) -> None:
        self._check(self.lib.bshmem_gpu_set_nvls(self.h, int(on)))

    def device_state(self) -> DevState:
        st = DevState()
        self._check(self.lib.bshmem_gpu_get_state(self.h, C.byref(st)))
        return st

    def check_error(self) -> None:
        self._check(self.lib.bshmem_gpu_check_error(self.h))

    def device_stats(self) -> dict:
        arr = (C.c_uint64 * len(DSTAT_NAMES))()
        self._check(self.lib.bshmem_gpu_get_device_stats(self.h, arr, len(DSTAT_NAMES)))
        return dict(zip(DSTAT_NAMES, (int(v) for v in arr)))

    def reset_device_stats(self) -> None:
        self._check(self.lib.bshmem_gpu_reset_device_stats(self.h))

    def trace_enable(self, capacity: int = 4096) -> None:
        """Record a device-side timeline of the last `capacity` (<= 16384) communication events; 0 switches it off.
        Needs profile=True (the default).  The reference only has counters (library/src/stats.hpp:121-145)."""
        self._check(self.lib.bshmem_gpu_trace_enable(self.h, capacity))

    def trace_events(self, max_events: int = 16384) -> list:
        """Events recorded since trace_enable(), oldest first: dicts of t_ns (%globaltimer), op, pe, block, bytes
        (for waits and barriers: the nanoseconds spent; for timeouts: the site code) and seq."""
        buf = (C.c_uint64 * (4 * max_events))()
        n, total = C.c_int(0), C.c_uint64(0)
        self._check(self.lib.bshmem_gpu_trace_read(self.h, buf, max_events, C.byref(n), C.byref(total)))
        out = []
        for k in range(n.value):
            t, w, b, seq = (int(buf[4 * k + i]) for i in range(4))
            out.append({"t_ns": t, "op": TRACE_OPS.get(w & 0xFF, str(w & 0xFF)), "pe": (w >> 8) & 0xFFFFFF, "block": w >> 32,
                        "bytes": b, "seq": seq})
        return out

    def rma_kernel(self, sym: torch.Tensor, local: torch.Tensor, pe: int, *, put: bool = True, scope: str = "block",
                   ctas: int = 32, threads: int = 512, nbytes: Optional[int] = None) -> None:
        """Device-initiated put/get striped over `ctas` CTAs (enqueued, not synchronised).  Scope "bulk" moves the
        data with bulk async copies through shared memory (16-byte aligned addresses and size)."""
        sc = {"thread": 0, "warp": 1, "block": 2, "bulk": 3}[scope]
        n = nbytes if nbytes is not None else local.numel() * local.element_size()
        self._check(self.lib.bshmem_gpu_rma_kernel(self.h, sym.data_ptr(), local.data_ptr(), n, pe, int(put), sc, ctas,
                                                   threads))

    def offset_of(self, t: torch.Tensor) -> int:
        return t.data_ptr() - int(self.lib.bshmem_heap_base(self.h))

    # ---- device-API micro-benchmarks / functional kernels (csrc/cuda/p2p_kernels.cu) ----
    def bench_amo_rate(self, target: torch.Tensor, peer: int, iters: int, ctas: int, threads: int) -> float:
        """8-byte fetch-adds from ctas x threads threads on distinct words of `peer`; returns million atomics / s."""
        ns = C.c_uint64(0)
        self._check(self.lib.bshmem_gpu_bench_amo_rate(self.h, target.data_ptr(), target.numel(), peer, iters, ctas, threads,
                                                       C.byref(ns)))
        return ctas * threads * iters / max(ns.value, 1) * 1e3

    def put_signal_stream(self, data: torch.Tensor, src: torch.Tensor, sig: torch.Tensor, nbytes: int, peer: int, iters: int,
                          ctas: int, threads: int = 512) -> None:
        """Enqueue `iters` one-way putmem_signal(ADD 1) of nbytes striped over ctas CTAs (not synchronised)."""
        self._check(self.lib.bshmem_gpu_put_signal_stream(self.h, data.data_ptr(), src.data_ptr(), sig.data_ptr(), nbytes, peer,
                                                          iters, ctas, threads))

    def bench_pingpong(self, flag: torch.Tensor, peer: int, iters: int, initiator: bool) -> float:
        """p + wait_until ping-pong with `peer`; returns one-way latency in microseconds."""
        ns = C.c_uint64(0)
        self._check(self.lib.bshmem_gpu_bench_pingpong(self.h, flag.data_ptr(), peer, iters, int(initiator), C.byref(ns)))
        return ns.value / iters / 2 / 1e3

    def bench_put_signal(self, data: torch.Tensor, sig: torch.Tensor, nbytes: int, peer: int, iters: int, initiator: bool,
                         threads: int = 512) -> float:
        ns = C.c_uint64(0)
        self._check(self.lib.bshmem_gpu_bench_put_signal(self.h, data.data_ptr(), sig.data_ptr(), nbytes, peer, iters,
                                                         int(initiator), threads, C.byref(ns)))
        return ns.value / iters / 2 / 1e3

    def bench_amo(self, target: torch.Tensor, peer: int, iters: int, op: int = D.AMO_FETCH_ADD) -> float:
        ns = C.c_uint64(0)
        self._check(self.lib.bshmem_gpu_bench_amo(self.h, target.data_ptr(), peer, iters, op, C.byref(ns)))
        return ns.value / iters / 1e3

    def bench_msgrate(self, dest: torch.Tensor, src: torch.Tensor, size: int, peer: int, windows: int, ctas: int,
                      threads: int) -> float:
        """put_nbi message rate (windows of 64 + quiet); returns million messages per second."""
        ns = C.c_uint64(0)
        self._check(self.lib.bshmem_gpu_bench_msgrate(self.h, dest.data_ptr(), src.data_ptr(), size, peer, windows, ctas,
                                                      threads, C.byref(ns)))
        return ctas * threads * 64 * windows / (ns.value * 1e-9) / 1e6

    def swarm_get(self, local: torch.Tensor, sym: torch.Tensor, size: int, peer: int, ctas: int, threads: int) -> None:
        self._check(self.lib.bshmem_gpu_swarm_get(self.h, local.data_ptr(), sym.data_ptr(), size, peer, ctas, threads))

    def api_selftest(self, peer: int) -> list[int]:
        """Runs the typed device API (p/g, all atomics, ptr, test) against `peer` inside one kernel."""
        si = self.zeros((4,), torch.int32)
        su = self.zeros((4,), torch.int64)
        sf = self.zeros((4,), torch.float32)
        res = torch.full((64,), -2, dtype=torch.int32, device=self.device)
        self._check(self.lib.bshmem_gpu_api_selftest(self.h, si.data_ptr(), su.data_ptr(), sf.data_ptr(), peer, res.data_ptr()))
        out = res.tolist()
        self.barrier_all()
        return out[:out.index(-1)]

    def bind_thread(self, ctx=None) -> None:
        """Run everything the calling thread issues from now on (collectives and waits included) on host context
        `ctx`'s stream, completing each call before it returns; None unbinds.  Used by service threads that must not
        queue behind the PE stream."""
        self._check(self.lib.bshmem_gpu_bind_thread_ctx(self.h, -1 if ctx is None else self._ctx(ctx)))

    def api_matrix_buffers(self, nbytes: int = 4096) -> dict:
        """Symmetric and local buffers of `api_matrix` (a collective allocation: every PE calls it)."""
        return {"si": self.zeros((4,), torch.int32), "su": self.zeros((4,), torch.int64), "sf": self.zeros((4,), torch.float32),
                "data": self.zeros((3 * nbytes,), torch.uint8), "coll": self.zeros((2 * 64 * 16,), torch.float32),
                "local": torch.zeros(6 * nbytes, dtype=torch.uint8, device=self.device), "nbytes": nbytes}

    def api_matrix(self, bufs: dict, team=None, peer: int = 0, proxy: bool = False) -> list[int]:
        """The device API matrix (p/g, 15 atomics, put/get at every scope, put_signal, fence/quiet, work-group
        collectives) through a context of `team` (None = world), PE numbers relative to that team; with `proxy` every
        operation goes through the reverse-offload ring.  Every member of the team must make the same call.
        Returns one 1/0 per check."""
        ring = None
        if proxy:
            if getattr(self, "proxy", None) is None:
                raise ShmemError(5, "api_matrix(proxy=True) needs a runtime initialised with backend='proxy'")
            ring = self.proxy.ring_dev
        for k in ("si", "su", "sf"):
            bufs[k].zero_()
        slot = 0 if team is None else team.slot
        res = torch.full((64,), -2, dtype=torch.int32, device=self.device)
        torch.cuda.synchronize(self.device)
        self._check(self.lib.bshmem_gpu_api_matrix(self.h, ring, slot, bufs["si"].data_ptr(), bufs["su"].data_ptr(),
                                                   bufs["sf"].data_ptr(), bufs["data"].data_ptr(), bufs["local"].data_ptr(),
                                                   bufs["coll"].data_ptr(), bufs["nbytes"], peer, res.data_ptr()))
        out = res.tolist()
        return out[:out.index(-1)]

    def global_exit(self, status: int = 0) -> None:
        """End the whole job with `status` (the reference calls MPI_Abort): publish the status in the bootstrap store —
        every other rank's watcher thread ends its process with it — and leave this process the same way."""
        w = getattr(self, "_exit_watcher", None)
        if w is not None:
            w.raise_exit(status)
        self.lib.bshmem_global_exit(self.h, int(status))
        os._exit(int(status) & 0xFF)

    def finalize(self) -> None:
        w = getattr(self, "_exit_watcher", None)
        if w is not None:
            w.stop()
        super().finalize()

    def functional_run(self, test_type: int, *, size: int, wgs: int, wg_size: int, loops: int, skip: int, peer: int, sym_a, sym_b,
                       local, words, timers, status, team=None, ctx_options: int = 0, initiator: bool = True,
                       n_bins: int = 0) -> float:
        """One launch of the functional tester's kernel for `test_type` (bench/functional.py holds the table of
        types and sizes the buffers); returns the CUDA-event time of the timed part in milliseconds."""
        ms = C.c_float(0.0)
        self._check(self.lib.bshmem_gpu_functional_run(
            self.h, test_type, 0 if team is None else team.slot, peer, wgs, wg_size, loops, skip, size, sym_a.data_ptr(),
            sym_b.data_ptr(), local.data_ptr(), words.data_ptr(), timers.data_ptr(), status.data_ptr(), ctx_options,
            1 if initiator else 0, n_bins, C.byref(ms)))
        return ms.value

    def wg_collectives(self, dst: torch.Tensor, src: torch.Tensor) -> int:
        st = C.c_int(-1)
        self._check(self.lib.bshmem_gpu_wg_collectives(self.h, dst.data_ptr(), src.data_ptr(), src.numel(), C.byref(st)))
        return st.value


def init_device_runtime(boot: Bootstrap, cfg: Config, device: Optional[int] = None, proxy: bool = False) -> DeviceRuntime:
    if not torch.cuda.is_available():
        raise ShmemError(7, "the device backend needs a CUDA device (use backend='cpu' otherwise)")
    lib = cuda_lib()
    if device is None:
        device = int(os.environ.get("LOCAL_RANK", boot.rank)) % torch.cuda.device_count()
    torch.cuda.set_device(device)
    torch.cuda.init()
    n = boot.world_size
    heap = C.c_void_p()
    mode = {"vmm": 0, "ipc": 1, "auto": 0}[cfg.heap_mode]
    st = lib.bshmem_gpu_heap_create(boot.rank, n, cfg.heap_bytes, device, mode, C.byref(heap))
    if st != 0 and cfg.heap_mode == "auto":
        mode = 1
        st = lib.bshmem_gpu_heap_create(boot.rank, n, cfg.heap_bytes, device, mode, C.byref(heap))
    _gpu_error(lib, "heap_create", st)
    # every PE must have picked the same mode
    modes = boot.allgather(mode, tag="heap-mode") if n > 1 else [mode]
    if len(set(modes)) != 1:
        raise ShmemError(7, f"PEs disagree on the heap mode: {modes}")
    if n > 1:
        if mode == 0:
            fd = C.c_int(-1)
            _gpu_error(lib, "heap_export_fd", lib.bshmem_gpu_heap_export_fd(heap, C.byref(fd)))
            fds = boot.exchange_fds([fd.value], tag="heap-fd")
            for pe in range(n):
                if pe != boot.rank:
                    _gpu_error(lib, f"heap_import_fd(pe {pe})", lib.bshmem_gpu_heap_import_fd(heap, pe, fds[pe][0]))
                    os.close(fds[pe][0])
            os.close(fd.value)
        else:
            buf = (C.c_char * 64)()
            _gpu_error(lib, "heap_export_ipc", lib.bshmem_gpu_heap_export_ipc(heap, buf))
            handles = boot.allgather(bytes(buf), tag="heap-ipc")
            for pe in range(n):
                if pe != boot.rank:
                    hb = (C.c_char * 64).from_buffer_copy(handles[pe])
                    _gpu_error(lib, f"heap_import_ipc(pe {pe})", lib.bshmem_gpu_heap_import_ipc(heap, pe, hb))
        boot.barrier("heap-mapped")
    nvls_on = False
    if n > 1 and mode == 0 and cfg.nvls in ("on", "auto"):
        sup = boot.allgather(int(lib.bshmem_gpu_multicast_supported(device)), tag="nvls-sup")
        if all(sup):
            fd = C.c_int(-1)
            if boot.rank == 0:
                _gpu_error(lib, "multicast_create", lib.bshmem_gpu_multicast_create(heap, C.byref(fd)))
            fds = boot.exchange_fds([fd.value] if boot.rank == 0 else [], tag="mc-fd")
            if boot.rank != 0:
                _gpu_error(lib, "multicast_import", lib.bshmem_gpu_multicast_import(heap, fds[0][0]))
                os.close(fds[0][0])
            else:
                os.close(fd.value)
            _gpu_error(lib, "multicast_add_device", lib.bshmem_gpu_multicast_add_device(heap))
            boot.barrier("mc-added")
            _gpu_error(lib, "multicast_bind", lib.bshmem_gpu_multicast_bind(heap))
            boot.barrier("mc-bound")
            nvls_on = True
        elif cfg.nvls == "on":
            raise ShmemError(8, "NVLink multicast requested but not supported on every PE")
    nc = native_config(cfg)
    nc.heap_bytes = lib.bshmem_gpu_heap_bytes(heap)
    h = C.c_void_p()
    _gpu_error(lib, "gpu_init", lib.bshmem_gpu_init(heap, C.byref(nc), cfg.coll_ctas, 1, C.byref(h)))
    rt = DeviceRuntime(lib, h.value, torch.device("cuda", device), heap)
    rt.config = cfg
    rt.bootstrap = boot
    rt.heap_mode = "vmm" if mode == 0 else "ipc"
    rt.nvls = nvls_on
    # Order the runtime's operations with the caller's PyTorch work: same stream as torch ops.
    rt.set_stream(torch.cuda.current_stream())
    if nvls_on:
        rt.set_nvls(True)
    if n > 1:
        boot.barrier("gpu-init")
        from .bootstrap import ExitWatcher
        rt._exit_watcher = ExitWatcher(boot)       # global_exit of any PE ends every PE
    if proxy:
        from .proxy import attach_proxy
        attach_proxy(rt)
    return rt


class LocalGroup:
    """All PEs of a job inside ONE process on ONE GPU — for tests on a single
    device.  Host RMA/atomics work per PE as usual; collectives and team splits
    run for the whole group at once (one cooperative launch), because kernels
    that wait on one another must never be separate launches on one GPU."""

    def __init__(self, n_pes: int, heap_bytes: int = 64 << 20, device: int = 0, config: Optional[Config] = None):
        self.lib = cuda_lib()
        self.n_pes = n_pes
        cfg = config or Config.from_env(backend="device", heap_bytes=heap_bytes)
        torch.cuda.set_device(device)
        torch.cuda.init()
        heaps = (C.c_void_p * n_pes)()
        _gpu_error(self.lib, "heap_create_local_group",
                   self.lib.bshmem_gpu_heap_create_local_group(n_pes, cfg.heap_bytes, device, heaps))
        self.heaps = list(heaps)
        self.pes: list[DeviceRuntime] = []
        nc = native_config(cfg)
        nc.heap_bytes = self.lib.bshmem_gpu_heap_bytes(self.heaps[0])
        for pe in range(n_pes):
            h = C.c_void_p()
            _gpu_error(self.lib, "gpu_init", self.lib.bshmem_gpu_init(self.heaps[pe], C.byref(nc), cfg.coll_ctas, 1, C.byref(h)))
            rt = DeviceRuntime(self.lib, h.value, torch.device("cuda", device), self.heaps[pe])
            rt.config = cfg
            rt.set_stream(torch.cuda.current_stream())
            self.pes.append(rt)
        self._handles = (C.c_void_p * n_pes)(*[rt.h.value for rt in self.pes])

    def empty(self, shape, dtype) -> list[torch.Tensor]:
        """The same symmetric allocation on every PE."""
        return [rt.empty(shape, dtype, collective=False) for rt in self.pes]

    def collective(self, kind: int, dests, srcs, count: int, *, dtype=None, op: int = 0, root: int = 0,
                   team_slot: int = 0, ctas: int = 2) -> None:
        d_off = self.pes[0].offset_of(dests[0]) if dests is not None else 0
        s_off = self.pes[0].offset_of(srcs[0]) if srcs is not None else 0
        code = D.code_of(dtype) if dtype is not None else 0
        st = self.lib.bshmem_gpu_group_collective(self._handles, self.n_pes, team_slot, kind, code, op, root, d_off, s_off,
                                                  count, ctas)
        _gpu_error(self.lib, "group_collective", st)

    def team_split(self, parent_slot: int, start: int, stride: int, size: int) -> list[int]:
        out = (C.c_int * self.n_pes)()
        _gpu_error(self.lib, "group_team_split",
                   self.lib.bshmem_gpu_group_team_split(self._handles, self.n_pes, parent_slot, start, stride, size, out))
        return list(out)

    def close(self) -> None:
        for rt in reversed(self.pes):
            if not rt.finalized:
                rt.finalize()
        self.pes = []
