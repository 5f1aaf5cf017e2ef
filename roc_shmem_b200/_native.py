"""ctypes bindings of the in-tree native libraries.

The libraries are plain ``extern "C"`` shared objects built by ``build.py`` into
``roc_shmem_b200/lib`` — no pybind/torch extension ABI, so they load in any
process (also C programs can link them).  Loading is lazy and fails loudly: a
GPU code path never falls back to eager PyTorch when its library is missing.
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from pathlib import Path

from . import build as _build

_LIB_DIR = Path(__file__).resolve().parent / "lib"
_lock = threading.Lock()
_libs: dict[str, C.CDLL] = {}


class NativeLibraryMissing(ImportError):
    pass


def load(name: str, *, build_if_missing: bool = True) -> C.CDLL:
    """Load ``lib/<name>``.  An existing library is used as it is: a multi-rank job imports this module in every
    rank at once, and ranks that each decided to recompile a library whose sources look newer would spend minutes
    in the compiler, racing on the same object files, before the first collective.  A missing library is built
    (one process at a time, under a file lock); set ``B200SHMEM_AUTO_REBUILD=1`` to also rebuild a stale one at
    import, as a developer convenience on a single process.  ``python -m roc_shmem_b200.build`` is the build step."""
    with _lock:
        if name in _libs:
            return _libs[name]
        path = _LIB_DIR / name
        want_build = build_if_missing and (not path.exists() or os.environ.get("B200SHMEM_AUTO_REBUILD", "") == "1")
        if want_build:
            try:
                with _build_lock():
                    if name == "libbshmem_host.so":
                        _build.build_host()
                    elif name in _build.CUDA_TARGETS:
                        _build.build_cuda_target(name)
            except Exception as e:   # keep an existing binary usable if the rebuild fails
                if not path.exists():
                    raise NativeLibraryMissing(f"cannot build {name}: {e}") from e
        if not path.exists():
            raise NativeLibraryMissing(f"{path} is missing; run `python -m roc_shmem_b200.build`")
        lib = C.CDLL(str(path), mode=C.RTLD_GLOBAL if name == "libbshmem_cuda.so" else C.RTLD_LOCAL)
        _libs[name] = lib
        return lib


class _build_lock:
    """Inter-process lock around an import-time build (ranks of one job share the source tree)."""

    def __enter__(self):
        import fcntl
        _LIB_DIR.mkdir(exist_ok=True)
        self._f = open(_LIB_DIR / ".build.lock", "w")
        fcntl.flock(self._f, fcntl.LOCK_EX)
        return self

    def __exit__(self, *exc):
        import fcntl
        fcntl.flock(self._f, fcntl.LOCK_UN)
        self._f.close()
        return False


class ErrorRecord(C.Structure):
    _fields_ = [("code", C.c_uint32), ("pe", C.c_int32), ("where", C.c_uint32), ("count", C.c_uint32),
                ("addr", C.c_uint64), ("expected", C.c_uint64), ("seen", C.c_uint64)]

    def as_dict(self) -> dict:
        return {k: getattr(self, k) for k, _ in self._fields_}


class NativeConfig(C.Structure):
    _fields_ = [("heap_bytes", C.c_uint64), ("timeout_us", C.c_uint64), ("max_teams", C.c_int32),
                ("max_ctxs", C.c_int32), ("debug", C.c_int32), ("profile", C.c_int32),
                ("requested_thread_level", C.c_int32), ("reserved0", C.c_int32)]


_VP, _I, _U64, _SZ, _L = C.c_void_p, C.c_int, C.c_uint64, C.c_size_t, C.c_long


def declare_runtime_api(lib: C.CDLL) -> None:
    """Argument/return types of the bshmem.h entry points (present in both the
    host library and the CUDA runtime library)."""
    def f(name, res, *args):
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = list(args)
    f("bshmem_config_default", None, C.POINTER(NativeConfig))
    f("bshmem_cpu_world_create", _I, C.c_char_p, _I, _U64, C.POINTER(_VP))
    f("bshmem_cpu_world_open", _I, C.c_char_p, C.POINTER(_VP))
    f("bshmem_cpu_world_destroy", _I, _VP)
    f("bshmem_cpu_world_mark_dead", _I, _VP, _I)
    f("bshmem_cpu_init", _I, _VP, _I, C.POINTER(NativeConfig), C.POINTER(_VP))
    f("bshmem_finalize", _I, _VP)
    f("bshmem_query_thread", _I, _VP, C.POINTER(_I))
    f("bshmem_my_pe", _I, _VP)
    f("bshmem_n_pes", _I, _VP)
    f("bshmem_global_exit", _I, _VP, _I)
    f("bshmem_last_error", C.c_char_p, _VP)
    f("bshmem_get_error_record", _I, _VP, C.POINTER(ErrorRecord), _I)
    f("bshmem_status_string", C.c_char_p, _I)
    f("bshmem_set_timeout_us", _I, _VP, _U64)
    f("bshmem_get_timeout_us", _U64, _VP)
    f("bshmem_set_current", None, _VP)
    f("bshmem_get_current", _VP)
    f("bshmem_malloc", _VP, _VP, _SZ)
    f("bshmem_align", _VP, _VP, _SZ, _SZ)
    f("bshmem_calloc", _VP, _VP, _SZ, _SZ)
    f("bshmem_free", _I, _VP, _VP)
    f("bshmem_malloc_local", _VP, _VP, _SZ, _SZ)
    f("bshmem_free_local", _I, _VP, _VP)
    f("bshmem_ptr", _VP, _VP, _VP, _I)
    f("bshmem_heap_base", _VP, _VP)
    f("bshmem_heap_bytes", _U64, _VP)
    f("bshmem_heap_usage", _I, _VP, C.POINTER(_U64 * 9))
    f("bshmem_addr_accessible", _I, _VP, _VP, _I)
    f("bshmem_ctx_create", _I, _VP, _L, C.POINTER(C.c_int32))
    f("bshmem_team_create_ctx", _I, _VP, C.c_int32, _L, C.POINTER(C.c_int32))
    f("bshmem_ctx_destroy", _I, _VP, C.c_int32)
    f("bshmem_team_split_strided", _I, _VP, C.c_int32, _I, _I, _I, C.POINTER(C.c_int32))
    f("bshmem_team_destroy", _I, _VP, C.c_int32)
    f("bshmem_team_n_pes", _I, _VP, C.c_int32)
    f("bshmem_team_my_pe", _I, _VP, C.c_int32)
    f("bshmem_team_translate_pe", _I, _VP, C.c_int32, _I, C.c_int32)
    for nm in ("putmem", "getmem", "putmem_nbi", "getmem_nbi"):
        f("bshmem_ctx_" + nm, _I, _VP, C.c_int32, _VP, _VP, _SZ, _I)
    for nm in ("putmem_signal", "putmem_signal_nbi"):
        f("bshmem_ctx_" + nm, _I, _VP, C.c_int32, _VP, _VP, _SZ, _VP, _U64, _I, _I)
    f("bshmem_signal_fetch", _U64, _VP, _VP)
    f("bshmem_ctx_amo", _I, _VP, C.c_int32, _I, _I, _VP, _U64, _U64, _I, C.POINTER(_U64))
    f("bshmem_ctx_fence", _I, _VP, C.c_int32)
    f("bshmem_ctx_quiet", _I, _VP, C.c_int32)
    f("bshmem_wait_until", _I, _VP, _I, _VP, _I, _U64)
    f("bshmem_test", _I, _VP, _I, _VP, _I, _U64, C.POINTER(_I))
    f("bshmem_barrier_all", _I, _VP)
    f("bshmem_sync_all", _I, _VP)
    f("bshmem_team_sync", _I, _VP, C.c_int32)
    f("bshmem_team_barrier", _I, _VP, C.c_int32)
    f("bshmem_team_broadcast", _I, _VP, C.c_int32, _VP, _VP, _SZ, _I)
    f("bshmem_team_reduce", _I, _VP, C.c_int32, _I, _I, _VP, _VP, _SZ)
    f("bshmem_team_reduce_scatter", _I, _VP, C.c_int32, _I, _I, _VP, _VP, _SZ)
    f("bshmem_team_reduce_root", _I, _VP, C.c_int32, _I, _I, _VP, _VP, _SZ, _I)
    f("bshmem_team_fcollect", _I, _VP, C.c_int32, _VP, _VP, _SZ)
    f("bshmem_team_alltoall", _I, _VP, C.c_int32, _VP, _VP, _SZ)
    f("bshmem_barrier", _I, _VP, _I, _I, _I, _VP)
    f("bshmem_sync", _I, _VP, _I, _I, _I, _VP)
    f("bshmem_broadcast", _I, _VP, _VP, _VP, _SZ, _I, _I, _I, _I, _VP)
    f("bshmem_to_all", _I, _VP, _I, _I, _VP, _VP, _SZ, _I, _I, _I, _VP, _VP)
    f("bshmem_stats_count", _I)
    f("bshmem_stats_name", C.c_char_p, _I)
    f("bshmem_get_stats", _I, _VP, C.POINTER(_U64), _I)
    f("bshmem_reset_stats", _I, _VP)
    f("bshmem_dump_stats", _I, _VP)


_host_declared = False


def host_lib() -> C.CDLL:
    global _host_declared
    lib = load("libbshmem_host.so")
    if not _host_declared:
        declare_runtime_api(lib)
        _host_declared = True
    return lib
