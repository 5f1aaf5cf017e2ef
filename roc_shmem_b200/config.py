"""Run-time configuration: defaults ← environment (``B200SHMEM_*``) ← kwargs.

The reference spreads its knobs over 14 CMake options and a dozen ``getenv``
calls (library/CMakeLists.txt:70-85; memory/single_heap.cpp:30 ROC_SHMEM_HEAP_SIZE,
team_tracker.cpp:31 ROC_SHMEM_MAX_NUM_TEAMS, host/host.cpp:106
ROC_SHMEM_MAX_NUM_HOST_CONTEXTS, reverse_offload/queue.cpp:31 RO_NET_CPU_QUEUE...).
Here there is one dataclass; the ``ROC_SHMEM_*`` spellings of the shared knobs are
accepted as aliases so existing job scripts keep working.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, fields


def _parse_size(v: str) -> int:
    v = v.strip().lower()
    mult = 1
    for suf, m in (("k", 1 << 10), ("m", 1 << 20), ("g", 1 << 30)):
        if v.endswith(suf + "ib"):
            v, mult = v[:-3], m
            break
        if v.endswith(suf + "b") or v.endswith(suf):
            v, mult = v.rstrip("b")[:-1], m
            break
    return int(float(v) * mult)


@dataclass
class Config:
    heap_bytes: int = 1 << 30          # symmetric heap per PE
    timeout_ms: int = 30_000           # bound of every blocking wait, host and device
    max_teams: int = 40                # incl. TEAM_WORLD
    max_ctxs: int = 40                 # host contexts
    debug: bool = False                # bounds checks, verbose native errors
    profile: bool = True               # API-call counters
    backend: str = "auto"              # auto | device | proxy | cpu
    nvls: str = "auto"                 # NVLink multicast object: off | on | auto (on where every PE supports it)
    heap_mode: str = "auto"            # auto | vmm | ipc (how peers' heaps get mapped)
    proxy_slots: int = 1024            # ring slots of the reverse-offload queue
    coll_ctas: int = 128               # CTAs per PE for host-launched collectives
    slab_bytes: int = 1 << 20          # device-callable slab allocator region

    _ALIASES = {
        "heap_bytes": ("B200SHMEM_HEAP_SIZE", "ROC_SHMEM_HEAP_SIZE"),
        "timeout_ms": ("B200SHMEM_TIMEOUT_MS",),
        "max_teams": ("B200SHMEM_MAX_NUM_TEAMS", "ROC_SHMEM_MAX_NUM_TEAMS"),
        "max_ctxs": ("B200SHMEM_MAX_NUM_HOST_CONTEXTS", "ROC_SHMEM_MAX_NUM_HOST_CONTEXTS"),
        "debug": ("B200SHMEM_DEBUG", "ROC_SHMEM_DEBUG"),
        "profile": ("B200SHMEM_PROFILE",),
        "backend": ("B200SHMEM_BACKEND",),
        "nvls": ("B200SHMEM_NVLS",),
        "heap_mode": ("B200SHMEM_HEAP_MODE",),
        "proxy_slots": ("B200SHMEM_PROXY_SLOTS", "RO_NET_QUEUE_SIZE"),
        "coll_ctas": ("B200SHMEM_COLL_CTAS", "ROC_SHMEM_NUM_BLOCKS"),
        "slab_bytes": ("B200SHMEM_SLAB_SIZE", "ROC_SHMEM_SLAB_SIZE"),
    }

    @classmethod
    def from_env(cls, **overrides) -> "Config":
        cfg = cls()
        for f in fields(cls):
            if f.name.startswith("_"):
                continue
            for env in cls._ALIASES.get(f.name, ()):
                if env in os.environ:
                    raw = os.environ[env]
                    if f.type in ("int", int):
                        val = _parse_size(raw)
                    elif f.type in ("bool", bool):
                        val = raw.strip().lower() not in ("", "0", "false", "off", "no")
                    else:
                        val = raw.strip().lower()
                    setattr(cfg, f.name, val)
                    break
        for k, v in overrides.items():
            if v is None:
                continue
            if not hasattr(cfg, k) or k.startswith("_"):
                raise TypeError(f"unknown config field {k!r}")
            setattr(cfg, k, v)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.heap_bytes < (1 << 16):
            raise ValueError("heap_bytes must be at least 64 KiB")
        if not 1 <= self.max_teams <= 40:
            raise ValueError("max_teams must be in [1, 40]")
        if not 1 <= self.max_ctxs <= 40:
            raise ValueError("max_ctxs must be in [1, 40]")
        if self.backend not in ("auto", "device", "proxy", "cpu"):
            raise ValueError(f"unknown backend {self.backend!r}")
        if self.nvls not in ("off", "on", "auto"):
            raise ValueError(f"nvls must be off/on/auto, not {self.nvls!r}")
        if self.heap_mode not in ("auto", "vmm", "ipc"):
            raise ValueError(f"heap_mode must be auto/vmm/ipc, not {self.heap_mode!r}")
        if self.proxy_slots < 2 or self.proxy_slots & (self.proxy_slots - 1):
            raise ValueError("proxy_slots must be a power of two >= 2")
