"""Host-side observability: a package logger controlled by ``B200SHMEM_DEBUG`` / ``B200SHMEM_LOG`` and NVTX
ranges around host paths (visible in any CUDA timeline tool) when ``B200SHMEM_TRACE=1``.

The reference prints with compile-time ``DPRINTF`` macros (library/src/util.hpp:101-121) and has no timeline
hooks; the device-side timeline lives in ``DeviceRuntime.trace_enable / trace_events``.
"""
from __future__ import annotations

import contextlib
import logging
import os

logger = logging.getLogger("roc_shmem_b200")
if not logger.handlers:
    _h = logging.StreamHandler()
    _h.setFormatter(logging.Formatter("[bshmem %(levelname)s pe=%(pe)s] %(message)s", defaults={"pe": "?"}))
    logger.addHandler(_h)
    level = os.environ.get("B200SHMEM_LOG", "").upper()
    if not level and os.environ.get("B200SHMEM_DEBUG", os.environ.get("ROC_SHMEM_DEBUG", "0")) not in ("", "0"):
        level = "DEBUG"
    logger.setLevel(getattr(logging, level, logging.WARNING) if level else logging.WARNING)
    logger.propagate = False

_TRACE = os.environ.get("B200SHMEM_TRACE", "0") not in ("", "0")


def tracing() -> bool:
    return _TRACE


def set_tracing(on: bool) -> None:
    global _TRACE
    _TRACE = bool(on)


@contextlib.contextmanager
def nvtx_range(name: str):
    """NVTX range around a host path; free when tracing is off or CUDA is absent."""
    if not _TRACE:
        yield
        return
    import torch
    if not torch.cuda.is_available():
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


def log(pe: int, msg: str, *args, level: int = logging.DEBUG) -> None:
    logger.log(level, msg, *args, extra={"pe": pe})


def traced(name: str):
    """Decorator: wrap a host API method in an NVTX range when tracing is on (a flag test otherwise)."""
    def deco(fn):
        def wrapper(*a, **k):
            if not _TRACE:
                return fn(*a, **k)
            with nvtx_range(name):
                return fn(*a, **k)
        wrapper.__name__, wrapper.__doc__ = fn.__name__, fn.__doc__
        return wrapper
    return deco


def instrument(cls, names) -> None:
    for n in names:
        if hasattr(cls, n):
            setattr(cls, n, traced(f"bshmem.{n}")(getattr(cls, n)))
