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


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=str(PKG.parent / "docs" / "api_reference.md"))
    a = ap.parse_args(argv)
    Path(a.out).parent.mkdir(parents=True, exist_ok=True)
    Path(a.out).write_text(generate())
    print(a.out)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
