"""API reference generator: walks the public headers (csrc/include) and writes one Markdown file with every
declaration and the comment that precedes it — the stand-in for the reference's doxygen target
(library/docs/CMakeLists.txt:23-38).

    python -m roc_shmem_b200.docs [--out docs/api_reference.md]
"""
from __future__ import annotations

import argparse
import re
from pathlib import Path

PKG = Path(__file__).resolve().parent
HEADERS = ["bshmem.h", "bshmem_types.h", "bshmem_typed.h", "bshmem_gpu.h", "bshmem_gpu_noalloc.h", "bshmem_proxy.h",
           "bshmem_device.cuh", "bshmem_coll.cuh", "bshmem_proxy_device.cuh", "bshmem_device_util.cuh"]

_DECL = re.compile(r"^\s*(?:template\s*<[^>]*>\s*)?(?:__device__\s+|__host__\s+|__forceinline__\s+|__noinline__\s+|static\s+|inline\s+|extern\s+)*"
                   r"[A-Za-z_][\w:<>,\s\*&]*?\s+\**([A-Za-z_]\w*)\s*\(([^;{]*)\)\s*(?:const\s*)?[;{]")


def _entries(text: str):
    """(name, signature, comment) for every function-like declaration at brace depth <= 2."""
    lines = text.splitlines()
    comment: list[str] = []
    i = 0
    while i < len(lines):
        ln = lines[i]
        s = ln.strip()
        if s.startswith("//"):
            comment.append(s.lstrip("/ ").rstrip())
        elif s.startswith("/*"):
            block = [s]
            while "*/" not in lines[i] and i + 1 < len(lines):
                i += 1
                block.append(lines[i].strip())
            comment = [b.strip("/* ").rstrip() for b in block]
        elif re.match(r"^BSHMEM_(DEV|PROXY)_CTX_AMO_(VALUE|NOVALUE)\((\w+),\s*(\w+)\)$", s):
            m = re.match(r"^BSHMEM_(DEV|PROXY)_CTX_AMO_(VALUE|NOVALUE)\((\w+),\s*(\w+)\)$", s)
            args = "T* dest, T value, int pe" if m.group(2) == "VALUE" else "T* dest, int pe"
            yield ("ctx_" + m.group(4), f"template <typename T> {m.group(3)} ctx_{m.group(4)}(const State& s, const Ctx& c, {args})",
                   "context form: the PE is relative to the context's team")
        elif re.match(r"^BSHMEM_DEV_BITWISE\((\w+),", s):
            nm = re.match(r"^BSHMEM_DEV_BITWISE\((\w+),", s).group(1)
            yield ("atomic_fetch_" + nm, f"template <typename T> T atomic_fetch_{nm}(const State& s, T* dest, T value, int pe)", "")
            yield ("atomic_" + nm, f"template <typename T> void atomic_{nm}(const State& s, T* dest, T value, int pe)", "")
        else:
            sig = s
            j = i
            while sig.count("(") > sig.count(")") and j + 1 < len(lines) and j - i < 6:
                j += 1
                sig += " " + lines[j].strip()
            m = _DECL.match(sig)
            if m and m.group(1) not in ("if", "for", "while", "switch", "return", "sizeof", "asm", "defined", "static_assert"):
                yield m.group(1), re.sub(r"\s+", " ", sig.split("{")[0].rstrip(" ;")), " ".join(c for c in comment if c)
            if s:
                comment = []
        i += 1


def generate() -> str:
    out = ["# bshmem API reference", "",
           "Generated from the headers under `roc_shmem_b200/csrc/include` by `python -m roc_shmem_b200.docs`.", ""]
    for h in HEADERS:
        path = PKG / "csrc" / "include" / h
        if not path.exists():
            continue
        text = path.read_text()
        out += [f"## {h}", ""]
        head = re.match(r"\s*((?://[^\n]*\n)+|/\*.*?\*/)", text, re.S)
        if head:
            out += [re.sub(r"^\s*(//|/\*|\*/|\*)\s?", "", ln) for ln in head.group(1).splitlines()] + [""]
        seen = set()
        for name, sig, comment in _entries(text):
            if (name, sig) in seen:
                continue
            seen.add((name, sig))
            out.append(f"* `{sig}`" + (f" — {comment}" if comment else ""))
        out.append("")
    return "\n".join(out)


# ---- porting guide: reference name -> name here ------------------------------------------------------------
# (reference name without the roc_shmem_ prefix) -> (host C entry or "", device function or "", Python or "", note)
PORTING = {
    "init": ("bshmem_cpu_init / bshmem_gpu_init", "", "roc_shmem_b200.init(backend)", "the backend is a run-time choice"),
    "init_thread": ("bshmem_cpu_init / bshmem_gpu_init (config.requested_thread_level)", "", "roc_shmem_b200.init_thread(level)", ""),
    "query_thread": ("bshmem_query_thread", "dev::query_thread", "Runtime.query_thread()", "always THREAD_MULTIPLE"),
    "finalize": ("bshmem_finalize", "", "roc_shmem_b200.finalize()", ""),
    "global_exit": ("bshmem_global_exit", "", "Runtime.global_exit(status)", ""),
    "my_pe": ("bshmem_my_pe", "dev::my_pe", "Runtime.my_pe", ""),
    "n_pes": ("bshmem_n_pes", "dev::n_pes", "Runtime.n_pes", ""),
    "malloc": ("bshmem_malloc", "", "Runtime.empty / zeros / malloc", "collective; symmetric tensors are the Python view"),
    "free": ("bshmem_free", "", "Runtime.free / free_ptr", ""),
    "ptr": ("bshmem_ptr", "dev::ptr", "Runtime.ptr(t, pe)", "every PE of a node is mapped, so never null on the device"),
    "putmem": ("bshmem_putmem", "dev::putmem<Scope>", "Runtime.put", "Scope = THREAD, WARP, BLOCK (the reference's _wave / _wg forms)"),
    "putmem_nbi": ("bshmem_putmem_nbi", "dev::putmem_nbi<Scope>", "Runtime.put(nbi=True)", ""),
    "getmem": ("bshmem_getmem", "dev::getmem<Scope>", "Runtime.get", ""),
    "getmem_nbi": ("bshmem_getmem_nbi", "dev::getmem_nbi<Scope>", "Runtime.get(nbi=True)", ""),
    "fence": ("bshmem_fence", "dev::fence", "Runtime.fence()", ""),
    "quiet": ("bshmem_quiet", "dev::quiet", "Runtime.quiet()", ""),
    "threadfence_system": ("", "dev::threadfence_system", "", ""),
    "barrier_all": ("bshmem_barrier_all", "coll::wg_barrier_all", "Runtime.barrier_all()", ""),
    "sync_all": ("bshmem_sync_all", "coll::wg_sync_all", "Runtime.sync_all()", ""),
    "wait": ("bshmem_wait_until", "dev::wait_until", "Runtime.wait_until", "bounded: returns BSHMEM_ERR_TIMEOUT instead of hanging"),
    "timer": ("", "dev::timer", "", "nanoseconds of %globaltimer"),
    "dump_stats": ("bshmem_dump_stats", "", "Runtime.dump_stats()", ""),
    "reset_stats": ("bshmem_reset_stats", "", "Runtime.reset_stats()", ""),
    "ctx_create": ("bshmem_ctx_create", "", "Runtime.ctx_create(options)", ""),
    "ctx_destroy": ("bshmem_ctx_destroy", "", "Context.destroy()", ""),
    "ctx_putmem": ("bshmem_ctx_putmem", "dev::ctx_putmem<Scope>", "Context.put", "PE numbers relative to the context's team"),
    "ctx_putmem_nbi": ("bshmem_ctx_putmem_nbi", "dev::ctx_putmem_nbi<Scope>", "Context.put(nbi=True)", ""),
    "ctx_getmem": ("bshmem_ctx_getmem", "dev::ctx_getmem<Scope>", "Context.get", ""),
    "ctx_getmem_nbi": ("bshmem_ctx_getmem_nbi", "dev::ctx_getmem_nbi<Scope>", "Context.get(nbi=True)", ""),
    "ctx_fence": ("bshmem_ctx_fence", "dev::ctx_fence", "Context.fence()", ""),
    "ctx_quiet": ("bshmem_ctx_quiet", "dev::ctx_quiet", "Context.quiet()", "completes that context's operations only"),
    "ctx_threadfence_system": ("", "dev::ctx_threadfence_system", "", ""),
    "ctx_my_pe": ("", "dev::ctx_my_pe", "Context.team.my_pe", ""),
    "ctx_n_pes": ("", "dev::ctx_n_pes", "Context.team.n_pes", ""),
    "wg_init": ("", "dev::wg_init", "", ""),
    "wg_init_thread": ("", "dev::wg_init_thread", "", ""),
    "wg_finalize": ("", "dev::wg_finalize", "", ""),
    "wg_ctx_create": ("", "dev::wg_ctx_create", "", "a device context is a value: option bits + team"),
    "wg_ctx_destroy": ("", "dev::wg_ctx_destroy", "", ""),
    "wg_team_create_ctx": ("", "dev::wg_team_create_ctx", "", ""),
    "wg_barrier_all": ("", "coll::wg_barrier_all", "", ""),
    "wg_sync_all": ("", "coll::wg_sync_all", "", ""),
    "wg_team_sync": ("", "coll::wg_team_sync", "", ""),
    "ctx_wg_barrier_all": ("", "coll::ctx_wg_barrier_all", "", ""),
    "ctx_wg_sync_all": ("", "coll::ctx_wg_sync_all", "", ""),
    "ctx_wg_team_sync": ("", "coll::ctx_wg_team_sync", "", ""),
    "team_split_strided": ("bshmem_team_split_strided", "", "Team.split_strided", ""),
    "team_destroy": ("bshmem_team_destroy", "", "Team.destroy()", ""),
    "team_my_pe": ("bshmem_team_my_pe", "", "Team.my_pe", ""),
    "team_n_pes": ("bshmem_team_n_pes", "", "Team.n_pes", ""),
    "team_translate_pe": ("bshmem_team_translate_pe", "dev::team_translate_pe", "Team.translate_pe", ""),
}
# typed families the reference generates with macros: (pattern there, pattern here on the host, on the device)
PORTING_FAMILIES = [
    ("roc_shmem_[ctx_]TYPE_put / get [_nbi]", "bshmem_[ctx_]TYPE_put / get [_nbi]", "dev::[ctx_]put / get [_nbi]<T, Scope>"),
    ("roc_shmem_[ctx_]TYPE_p / g", "bshmem_[ctx_]TYPE_p / g", "dev::[ctx_]p / g<T>"),
    ("roc_shmem_[ctx_]TYPE_atomic_{fetch_add, fetch_inc, fetch, compare_swap, swap, set, add, inc, fetch_and, fetch_or, fetch_xor, and, or, xor}",
     "bshmem_[ctx_]TYPE_atomic_*", "dev::[ctx_]atomic_*<T> (all 15 on the device)"),
    ("roc_shmem_TYPE_wait_until / test", "bshmem_TYPE_wait_until / test", "dev::wait_until / test<T> (bounded)"),
    ("roc_shmem_[ctx_]TYPE_OP_wg_to_all (team and active-set forms)", "bshmem_TYPE_OP_to_all, bshmem_team_reduce, bshmem_team_reduce_root, bshmem_team_reduce_scatter",
     "coll::[ctx_]wg_to_all<T>, coll::team_reduce / team_reduce_root / team_reduce_scatter<T>"),
    ("roc_shmem_[ctx_]TYPE_wg_broadcast / alltoall / fcollect", "bshmem_TYPE_broadcast / alltoall / fcollect, bshmem_team_*",
     "coll::[ctx_]wg_broadcast / wg_alltoall / wg_fcollect<T>"),
    ("— (not in the reference; OpenSHMEM 1.5)", "bshmem_[ctx_]putmem_signal[_nbi], bshmem_[ctx_]TYPE_put_signal[_nbi], bshmem_signal_fetch",
     "dev::[ctx_]putmem_signal<Scope>, dev::signal_fetch"),
]


def _header_text() -> str:
    return "\n".join((PKG / "csrc" / "include" / h).read_text() for h in HEADERS if (PKG / "csrc" / "include" / h).exists())


def porting_targets_missing() -> list[str]:
    """Names on the right-hand side of PORTING that no public header declares (a test keeps this list empty)."""
    text = _header_text()
    missing = []
    for ref, (host, device, _py, _note) in PORTING.items():
        for target in (host, device):
            for name in re.findall(r"(?:bshmem_|dev::|coll::)(\w+)", target):
                full = ("bshmem_" + name) if "bshmem_" + name in target else name
                if not re.search(r"\b" + re.escape(full) + r"\b", text):
                    missing.append(f"{ref} -> {full}")
    return missing


def porting_guide() -> str:
    out = ["# Moving from ROC_SHMEM to bshmem", "",
           "Generated by `python -m roc_shmem_b200.docs`.  Left: the name in the reference's public header",
           "(`library/include/roc_shmem.hpp`, prefix `roc_shmem_` dropped); right: what to call here.  Host C entries take the",
           "runtime handle first (handle-free typed names live in `bshmem_typed.h`); device functions live in",
           "`bshmem::dev` / `bshmem::coll` and take the `State` the kernel was given by value.", "",
           "| reference | host C | device | Python | note |", "|---|---|---|---|---|"]
    for ref, (host, device, py, note) in PORTING.items():
        out.append(f"| `{ref}` | {('`' + host + '`') if host else '—'} | {('`' + device + '`') if device else '—'} | "
                   f"{('`' + py + '`') if py else '—'} | {note} |")
    out += ["", "## Typed families", "", "| reference | host C | device |", "|---|---|---|"]
    for ref, host, device in PORTING_FAMILIES:
        out.append(f"| `{ref}` | `{host}` | `{device}` |")
    out += ["", "Option bits (`ROC_SHMEM_CTX_*` → `BSHMEM_CTX_*`), comparison and reduction operator codes, `ROC_SHMEM_TEAM_WORLD`,",
            "the active-set scratch sizes and the environment variables (`ROC_SHMEM_HEAP_SIZE`, `ROC_SHMEM_MAX_NUM_TEAMS`, …, also",
            "accepted under the `B200SHMEM_` prefix) keep their values and meaning.", ""]
    return "\n".join(out)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=str(PKG.parent / "docs" / "api_reference.md"))
    a = ap.parse_args(argv)
    Path(a.out).parent.mkdir(parents=True, exist_ok=True)
    Path(a.out).write_text(generate())
    guide = Path(a.out).parent / "porting_from_roc_shmem.md"
    guide.write_text(porting_guide())
    print(a.out)
    print(guide)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
