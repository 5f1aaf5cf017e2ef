"""Where the headers and libraries are, for C / C++ / CUDA users of the runtime (a pkg-config stand-in).

    bshmem-config --includedir | --libdir | --cmakedir | --cflags | --libs [--cuda]

The reference installs ``librocshmem.a`` plus a CMake package (library/CMakeLists.txt:90-295); here the libraries
are shared objects built in place, and this tool (or ``cmake/bshmemConfig.cmake``) tells a build where they are.
"""
from __future__ import annotations

import argparse
from pathlib import Path

PKG = Path(__file__).resolve().parent


def paths() -> dict[str, Path]:
    return {"includedir": PKG / "csrc" / "include", "libdir": PKG / "lib", "cmakedir": PKG / "cmake"}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    for k in ("includedir", "libdir", "cmakedir", "cflags", "libs", "cuda"):
        ap.add_argument("--" + k, action="store_true")
    a = ap.parse_args(argv)
    p = paths()
    out = []
    if a.includedir:
        out.append(str(p["includedir"]))
    if a.libdir:
        out.append(str(p["libdir"]))
    if a.cmakedir:
        out.append(str(p["cmakedir"]))
    if a.cflags:
        out.append(f"-I{p['includedir']}")
    if a.libs:
        lib = "bshmem_cuda" if a.cuda else "bshmem_host"
        out.append(f"-L{p['libdir']} -Wl,-rpath,{p['libdir']} -l{lib}")
    print(" ".join(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
