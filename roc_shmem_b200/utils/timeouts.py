"""Temporarily tighten the bound of blocking waits (used by failure-detection tests)."""
from __future__ import annotations

import contextlib


@contextlib.contextmanager
def temporary_timeout(rt, timeout_ms: int):
    """Within the block every blocking wait of `rt` gives up after `timeout_ms`."""
    old = rt.lib.bshmem_get_timeout_us(rt.h)
    rt.lib.bshmem_set_timeout_us(rt.h, timeout_ms * 1000)
    try:
        yield
    finally:
        rt.lib.bshmem_set_timeout_us(rt.h, old)
