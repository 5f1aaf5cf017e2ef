"""The per-PE runtime object: OpenSHMEM-style host API over a native handle.

One ``Runtime`` is one PE.  It is backend-agnostic: the CPU backend (threads or
processes over shared memory) and the NVLink backend (one process per GPU)
expose the same C entry points, so this class only differs in how a symmetric
allocation is wrapped into a ``torch.Tensor``.

API-shape parity: the host functions of library/include/roc_shmem.hpp:144-460
(init/finalize, malloc/free, contexts, teams, put/get(+nbi), p/g, the atomic
families, fence/quiet, wait_until/test, barrier/sync, broadcast, to_all) plus
the extensions the reference lacks (putmem_signal, reduce_scatter, host
fcollect/alltoall).  Typed names collapse into dtype-generic methods because the
tensors carry their dtype.
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, Optional, Sequence

import torch

from . import _native
from .utils import dtypes as D
from .utils.errors import ShmemError, raise_for_status

TEAM_WORLD = 0
TEAM_INVALID = -1
CTX_DEFAULT = 0

CTX_NOSTORE, CTX_SERIALIZED, CTX_WG_PRIVATE, CTX_SHARED = 1, 2, 4, 8


def _ptr_of(x) -> int:
    """Raw address of a tensor / numpy array / int."""
    if isinstance(x, torch.Tensor):
        return x.data_ptr()
    if isinstance(x, int):
        return x
    if hasattr(x, "ctypes"):
        return x.ctypes.data
    raise TypeError(f"cannot take the address of {type(x)}")


def _nbytes(x) -> int:
    if isinstance(x, torch.Tensor):
        return x.numel() * x.element_size()
    return x.nbytes


class Team:
    """A strided PE subset; slot 0 is TEAM_WORLD."""

    def __init__(self, rt: "Runtime", slot: int):
        self.rt, self.slot = rt, slot

    @property
    def valid(self) -> bool:
        return self.slot >= 0

    @property
    def n_pes(self) -> int:
        return self.rt.lib.bshmem_team_n_pes(self.rt.h, self.slot)

    @property
    def my_pe(self) -> int:
        return self.rt.lib.bshmem_team_my_pe(self.rt.h, self.slot)

    def translate_pe(self, pe: int, dest: "Team") -> int:
        return self.rt.lib.bshmem_team_translate_pe(self.rt.h, self.slot, pe, dest.slot)

    def split_strided(self, start: int, stride: int, size: int) -> "Team":
        return self.rt.team_split_strided(self, start, stride, size)

    def destroy(self) -> None:
        if self.slot > 0:
            raise_for_status(self.rt.lib.bshmem_team_destroy(self.rt.h, self.slot))
            self.slot = TEAM_INVALID

    def sync(self) -> None:
        self.rt._check(self.rt.lib.bshmem_team_sync(self.rt.h, self.slot))

    def barrier(self) -> None:
        self.rt._check(self.rt.lib.bshmem_team_barrier(self.rt.h, self.slot))

    def __repr__(self) -> str:
        return f"Team(slot={self.slot}, my_pe={self.my_pe}, n_pes={self.n_pes})"


class Context:
    """A host communication context (ordering domain + statistics); PE numbers
    passed with it are relative to the team it was created on."""

    def __init__(self, rt: "Runtime", idx: int, options: int, team: Team):
        self.rt, self.idx, self.options, self.team = rt, idx, options, team

    def destroy(self) -> None:
        if self.idx > 0:
            raise_for_status(self.rt.lib.bshmem_ctx_destroy(self.rt.h, self.idx))
            self.idx = -1

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.destroy()

    # convenience forwards
    def put(self, dest, src, pe, **kw):
        return self.rt.put(dest, src, pe, ctx=self, **kw)

    def get(self, dest, src, pe, **kw):
        return self.rt.get(dest, src, pe, ctx=self, **kw)

    def fence(self):
        self.rt.fence(self)

    def quiet(self):
        self.rt.quiet(self)

    def put_signal(self, dest, src, sig, value, pe, **kw):
        return self.rt.put_signal(dest, src, sig, value, pe, ctx=self, **kw)

    def __getattr__(self, name):
        # the atomic family: ctx.atomic_fetch_add(dest, value, pe) == rt.atomic_fetch_add(dest, value, pe, ctx=ctx)
        if name.startswith("atomic_"):
            fn = getattr(self.rt, name)
            return lambda *a, **kw: fn(*a, ctx=self, **kw)
        raise AttributeError(name)


class Runtime:
    def __init__(self, lib: C.CDLL, handle: int, *, tensor_from_ptr: Callable, device: torch.device,
                 on_finalize: Optional[Callable] = None):
        self.lib = lib
        self.h = C.c_void_p(handle)
        self._tensor_from_ptr = tensor_from_ptr
        self.device = device
        self._on_finalize = on_finalize
        self.my_pe = lib.bshmem_my_pe(self.h)
        self.n_pes = lib.bshmem_n_pes(self.h)
        self.team_world = Team(self, TEAM_WORLD)
        self.ctx_default = Context(self, CTX_DEFAULT, 0, self.team_world)
        self._live: dict[int, torch.Tensor] = {}
        self.finalized = False

    # ---- plumbing -------------------------------------------------------
    def _check(self, status: int) -> None:
        if status != 0:
            detail = self.lib.bshmem_last_error(self.h)
            raise_for_status(status, detail.decode() if detail else "")

    def _ctx(self, ctx) -> int:
        return CTX_DEFAULT if ctx is None else (ctx.idx if isinstance(ctx, Context) else int(ctx))

    def _team(self, team) -> int:
        return TEAM_WORLD if team is None else (team.slot if isinstance(team, Team) else int(team))

    def make_current(self) -> None:
        """Bind this PE to the calling thread for the handle-free typed C API."""
        self.lib.bshmem_set_current(self.h)

    # ---- lifecycle --------------------------------------------------------
    def finalize(self) -> None:
        if self.finalized:
            return
        self.finalized = True
        self._live.clear()
        st = self.lib.bshmem_finalize(self.h)
        if self._on_finalize:
            self._on_finalize()
        raise_for_status(st)

    def query_thread(self) -> int:
        out = C.c_int(0)
        self._check(self.lib.bshmem_query_thread(self.h, C.byref(out)))
        return out.value

    def global_exit(self, status: int = 0) -> None:
        """Flag the whole job as aborted; peers' waits return ShmemAborted."""
        self.lib.bshmem_global_exit(self.h, int(status))

    def error_record(self, clear: bool = True) -> dict:
        rec = _native.ErrorRecord()
        self._check(self.lib.bshmem_get_error_record(self.h, C.byref(rec), 1 if clear else 0))
        return rec.as_dict()

    # ---- symmetric memory ----------------------------------------------------
    def malloc(self, nbytes: int, align: int = 128) -> int:
        """Collective: returns the local address (0 for size 0 / exhaustion)."""
        p = self.lib.bshmem_align(self.h, align, nbytes)
        return int(p or 0)

    def free_ptr(self, ptr: int) -> None:
        self._check(self.lib.bshmem_free(self.h, C.c_void_p(ptr)))

    def empty(self, shape, dtype=torch.float32, *, align: int = 128, collective: bool = True) -> torch.Tensor:
        """Symmetric tensor: same offset in every PE's heap.  All PEs must call
        with the same sizes in the same order (that is what makes it symmetric)."""
        if isinstance(shape, int):
            shape = (shape,)
        shape = tuple(int(s) for s in shape)
        n = 1
        for s in shape:
            n *= s
        code = D.code_of(dtype)
        nbytes = max(n * D.size_of(code), 1)
        if collective:
            ptr = self.lib.bshmem_align(self.h, align, nbytes)
        else:
            ptr = self.lib.bshmem_malloc_local(self.h, nbytes, align)
        if not ptr:
            raise ShmemError(2, f"symmetric heap exhausted allocating {nbytes} bytes")
        t = self._tensor_from_ptr(int(ptr), shape, dtype)
        self._live[t.data_ptr()] = t
        return t

    def zeros(self, shape, dtype=torch.float32, **kw) -> torch.Tensor:
        t = self.empty(shape, dtype, collective=False, **kw)
        t.zero_()
        self.barrier_all()
        return t

    def free(self, t: torch.Tensor, *, collective: bool = True) -> None:
        ptr = t.data_ptr()
        self._live.pop(ptr, None)
        if collective:
            self._check(self.lib.bshmem_free(self.h, C.c_void_p(ptr)))
        else:
            self._check(self.lib.bshmem_free_local(self.h, C.c_void_p(ptr)))

    def ptr(self, t, pe: int) -> int:
        """Address of `t` in PE `pe`'s heap as mapped into this process (0 if not mapped)."""
        return int(self.lib.bshmem_ptr(self.h, C.c_void_p(_ptr_of(t)), pe) or 0)

    def peer_view(self, t: torch.Tensor, pe: int) -> torch.Tensor:
        """A tensor aliasing PE `pe`'s copy of the symmetric tensor `t`."""
        p = self.ptr(t, pe)
        if not p:
            raise ShmemError(4, "peer heap is not mapped")
        v = self._tensor_from_ptr(p, (t.numel(),), t.dtype)
        return v.as_strided(t.size(), t.stride())

    def heap_usage(self) -> dict:
        out = (C.c_uint64 * 9)()
        self._check(self.lib.bshmem_heap_usage(self.h, C.byref(out)))
        keys = ("heap_bytes", "reserved_bytes", "allocated_bytes", "requested_bytes", "live_blocks", "largest_free",
                "n_allocs", "n_frees", "n_failed")
        return dict(zip(keys, (int(v) for v in out)))

    def is_symmetric(self, t) -> bool:
        return bool(self.lib.bshmem_addr_accessible(self.h, C.c_void_p(_ptr_of(t)), self.my_pe))

    # ---- contexts / teams --------------------------------------------------------
    def ctx_create(self, options: int = 0, team: Optional[Team] = None) -> Context:
        out = C.c_int32(-1)
        tm = team or self.team_world
        self._check(self.lib.bshmem_team_create_ctx(self.h, tm.slot, options, C.byref(out)))
        return Context(self, out.value, options, tm)

    def team_split_strided(self, parent: Optional[Team], start: int, stride: int, size: int) -> Team:
        out = C.c_int32(-1)
        self._check(self.lib.bshmem_team_split_strided(self.h, self._team(parent), start, stride, size, C.byref(out)))
        return Team(self, out.value)

    # ---- RMA -----------------------------------------------------------------------
    def put(self, dest, src, pe: int, *, ctx=None, nbi: bool = False, nbytes: Optional[int] = None) -> None:
        """Copy `src` (any local buffer) into `dest`'s location on PE `pe`."""
        n = _nbytes(src) if nbytes is None else nbytes
        fn = self.lib.bshmem_ctx_putmem_nbi if nbi else self.lib.bshmem_ctx_putmem
        self._check(fn(self.h, self._ctx(ctx), _ptr_of(dest), _ptr_of(src), n, pe))

    def get(self, dest, src, pe: int, *, ctx=None, nbi: bool = False, nbytes: Optional[int] = None) -> None:
        """Copy `src`'s location on PE `pe` into the local buffer `dest`."""
        n = _nbytes(dest) if nbytes is None else nbytes
        fn = self.lib.bshmem_ctx_getmem_nbi if nbi else self.lib.bshmem_ctx_getmem
        self._check(fn(self.h, self._ctx(ctx), _ptr_of(dest), _ptr_of(src), n, pe))

    def put_signal(self, dest, src, sig, value: int, pe: int, *, op: int = D.SIGNAL_SET, ctx=None,
                   nbi: bool = False) -> None:
        """Put, then update the 64-bit signal word `sig` on PE `pe` (SET or ADD);
        the payload is visible to a reader that observed the signal."""
        fn = self.lib.bshmem_ctx_putmem_signal_nbi if nbi else self.lib.bshmem_ctx_putmem_signal
        self._check(fn(self.h, self._ctx(ctx), _ptr_of(dest), _ptr_of(src), _nbytes(src), _ptr_of(sig), value, op, pe))

    def signal_fetch(self, sig) -> int:
        return int(self.lib.bshmem_signal_fetch(self.h, _ptr_of(sig)))

    def p(self, dest: torch.Tensor, value, pe: int, *, ctx=None) -> None:
        """Single-element put of a scalar into dest[0] on PE `pe`."""
        code = D.code_of(dest.dtype)
        buf = (C.c_uint64 * 1)(D.to_bits(code, value))
        self._check(self.lib.bshmem_ctx_putmem_nbi(self.h, self._ctx(ctx), _ptr_of(dest), C.addressof(buf),
                                                   D.size_of(code), pe))

    def g(self, src: torch.Tensor, pe: int, *, ctx=None):
        """Single-element get of src[0] from PE `pe`."""
        code = D.code_of(src.dtype)
        buf = (C.c_uint64 * 1)(0)
        self._check(self.lib.bshmem_ctx_getmem(self.h, self._ctx(ctx), C.addressof(buf), _ptr_of(src),
                                               D.size_of(code), pe))
        return D.from_bits(code, buf[0])

    # ---- atomics ---------------------------------------------------------------------
    def _amo(self, op: int, dest: torch.Tensor, value, cond, pe: int, ctx) -> object:
        code = D.code_of(dest.dtype)
        fetched = C.c_uint64(0)
        self._check(self.lib.bshmem_ctx_amo(self.h, self._ctx(ctx), code, op, _ptr_of(dest), D.to_bits(code, value),
                                            D.to_bits(code, cond), pe, C.byref(fetched)))
        return D.from_bits(code, fetched.value)

    def atomic_fetch_add(self, dest, value, pe, ctx=None): return self._amo(D.AMO_FETCH_ADD, dest, value, 0, pe, ctx)
    def atomic_fetch_inc(self, dest, pe, ctx=None): return self._amo(D.AMO_FETCH_INC, dest, 0, 0, pe, ctx)
    def atomic_fetch(self, dest, pe, ctx=None): return self._amo(D.AMO_FETCH, dest, 0, 0, pe, ctx)
    def atomic_compare_swap(self, dest, cond, value, pe, ctx=None): return self._amo(D.AMO_FETCH_CSWAP, dest, value, cond, pe, ctx)
    def atomic_add(self, dest, value, pe, ctx=None): self._amo(D.AMO_ADD, dest, value, 0, pe, ctx)
    def atomic_inc(self, dest, pe, ctx=None): self._amo(D.AMO_INC, dest, 0, 0, pe, ctx)
    def atomic_cswap(self, dest, cond, value, pe, ctx=None): self._amo(D.AMO_CSWAP, dest, value, cond, pe, ctx)
    def atomic_set(self, dest, value, pe, ctx=None): self._amo(D.AMO_SET, dest, value, 0, pe, ctx)
    def atomic_swap(self, dest, value, pe, ctx=None): return self._amo(D.AMO_SWAP, dest, value, 0, pe, ctx)
    def atomic_fetch_and(self, dest, value, pe, ctx=None): return self._amo(D.AMO_FETCH_AND, dest, value, 0, pe, ctx)
    def atomic_fetch_or(self, dest, value, pe, ctx=None): return self._amo(D.AMO_FETCH_OR, dest, value, 0, pe, ctx)
    def atomic_fetch_xor(self, dest, value, pe, ctx=None): return self._amo(D.AMO_FETCH_XOR, dest, value, 0, pe, ctx)
    def atomic_and(self, dest, value, pe, ctx=None): self._amo(D.AMO_AND, dest, value, 0, pe, ctx)
    def atomic_or(self, dest, value, pe, ctx=None): self._amo(D.AMO_OR, dest, value, 0, pe, ctx)
    def atomic_xor(self, dest, value, pe, ctx=None): self._amo(D.AMO_XOR, dest, value, 0, pe, ctx)

    # ---- ordering / sync ------------------------------------------------------------------
    def fence(self, ctx=None) -> None:
        self._check(self.lib.bshmem_ctx_fence(self.h, self._ctx(ctx)))

    def quiet(self, ctx=None) -> None:
        self._check(self.lib.bshmem_ctx_quiet(self.h, self._ctx(ctx)))

    def wait_until(self, ivar: torch.Tensor, cmp, value) -> None:
        code = D.code_of(ivar.dtype)
        c = D.CMPS[cmp] if isinstance(cmp, str) else int(cmp)
        self._check(self.lib.bshmem_wait_until(self.h, code, _ptr_of(ivar), c, D.to_bits(code, value)))

    def test(self, ivar: torch.Tensor, cmp, value) -> bool:
        code = D.code_of(ivar.dtype)
        c = D.CMPS[cmp] if isinstance(cmp, str) else int(cmp)
        out = C.c_int(0)
        self._check(self.lib.bshmem_test(self.h, code, _ptr_of(ivar), c, D.to_bits(code, value), C.byref(out)))
        return bool(out.value)

    # ---- collectives -----------------------------------------------------------------------
    def barrier_all(self) -> None:
        self._check(self.lib.bshmem_barrier_all(self.h))

    def sync_all(self) -> None:
        self._check(self.lib.bshmem_sync_all(self.h))

    def broadcast(self, dest: torch.Tensor, src: torch.Tensor, root: int, team=None) -> None:
        """Root's `src` lands in every other member's `dest` (the root's own dest is untouched)."""
        self._check(self.lib.bshmem_team_broadcast(self.h, self._team(team), _ptr_of(dest), _ptr_of(src), _nbytes(src), root))

    def reduce(self, dest: torch.Tensor, src: torch.Tensor, op="sum", team=None) -> None:
        """Allreduce (`*_to_all`): every member gets op over all members' `src`; dest may alias src."""
        o = D.OPS[op] if isinstance(op, str) else int(op)
        self._check(self.lib.bshmem_team_reduce(self.h, self._team(team), D.code_of(src.dtype), o, _ptr_of(dest),
                                                _ptr_of(src), src.numel()))

    to_all = reduce

    def reduce_root(self, dest: torch.Tensor, src: torch.Tensor, root: int, op="sum", team=None) -> None:
        """Rooted reduce: only member `root` of the team gets op over all members' `src` (the others' dest is untouched)."""
        o = D.OPS[op] if isinstance(op, str) else int(op)
        self._check(self.lib.bshmem_team_reduce_root(self.h, self._team(team), D.code_of(src.dtype), o, _ptr_of(dest),
                                                     _ptr_of(src), src.numel(), root))

    def reduce_scatter(self, dest: torch.Tensor, src: torch.Tensor, op="sum", team=None) -> None:
        """dest (n elems) = op over members of their src[my_idx*n:(my_idx+1)*n]."""
        o = D.OPS[op] if isinstance(op, str) else int(op)
        self._check(self.lib.bshmem_team_reduce_scatter(self.h, self._team(team), D.code_of(src.dtype), o, _ptr_of(dest),
                                                        _ptr_of(src), dest.numel()))

    def fcollect(self, dest: torch.Tensor, src: torch.Tensor, team=None) -> None:
        """All-gather: my `src` lands in block my_idx of every member's `dest`."""
        self._check(self.lib.bshmem_team_fcollect(self.h, self._team(team), _ptr_of(dest), _ptr_of(src), _nbytes(src)))

    def alltoall(self, dest: torch.Tensor, src: torch.Tensor, team=None) -> None:
        """Block j of my `src` lands in block my_idx of member j's `dest`."""
        tm = self._team(team)
        n = self.lib.bshmem_team_n_pes(self.h, tm)
        self._check(self.lib.bshmem_team_alltoall(self.h, tm, _ptr_of(dest), _ptr_of(src), _nbytes(src) // max(n, 1)))

    # legacy active-set forms ------------------------------------------------------------------
    def barrier_active_set(self, pe_start: int, log_stride: int, pe_size: int, psync: torch.Tensor) -> None:
        self._check(self.lib.bshmem_barrier(self.h, pe_start, log_stride, pe_size, _ptr_of(psync)))

    def sync_active_set(self, pe_start: int, log_stride: int, pe_size: int, psync: torch.Tensor) -> None:
        self._check(self.lib.bshmem_sync(self.h, pe_start, log_stride, pe_size, _ptr_of(psync)))

    def broadcast_active_set(self, dest, src, root, pe_start, log_stride, pe_size, psync) -> None:
        self._check(self.lib.bshmem_broadcast(self.h, _ptr_of(dest), _ptr_of(src), _nbytes(src), root, pe_start,
                                              log_stride, pe_size, _ptr_of(psync)))

    def to_all_active_set(self, dest, src, op, pe_start, log_stride, pe_size, pwrk, psync) -> None:
        o = D.OPS[op] if isinstance(op, str) else int(op)
        self._check(self.lib.bshmem_to_all(self.h, D.code_of(src.dtype), o, _ptr_of(dest), _ptr_of(src), src.numel(),
                                           pe_start, log_stride, pe_size, _ptr_of(pwrk) if pwrk is not None else 0,
                                           _ptr_of(psync)))

    # ---- statistics ----------------------------------------------------------------------------
    def stats(self) -> dict:
        n = self.lib.bshmem_stats_count()
        arr = (C.c_uint64 * n)()
        self._check(self.lib.bshmem_get_stats(self.h, arr, n))
        return {self.lib.bshmem_stats_name(i).decode(): int(arr[i]) for i in range(n)}

    def reset_stats(self) -> None:
        self._check(self.lib.bshmem_reset_stats(self.h))

    def dump_stats(self) -> None:
        self._check(self.lib.bshmem_dump_stats(self.h))


# NVTX ranges around the host API when B200SHMEM_TRACE=1 (utils/trace.py)
from .utils.trace import instrument as _instrument  # noqa: E402

_instrument(Runtime, ("put", "get", "put_signal", "barrier_all", "sync_all", "quiet", "fence", "wait_until", "broadcast", "reduce",
                      "reduce_scatter", "fcollect", "alltoall", "malloc", "free", "team_split_strided", "ctx_create"))
