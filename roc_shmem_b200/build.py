"""In-tree build of the native libraries (no setuptools, no JIT cache).

Two kinds of artefacts land in ``roc_shmem_b200/lib``:

* ``libbshmem_host.so`` — pure C++17 (g++): allocator, teams, contexts, CPU
  backend, reverse-offload ring and service thread, typed C API.
* ``libbshmem_*.so`` built by nvcc for sm_100a: the NVLink runtime (CUDA VMM
  heap, device API kernels, collectives) and the tcgen05 GEMM / fused kernels.

The reference builds one static library with 14 CMake options
(library/CMakeLists.txt:70-85); here the backend is a run-time choice, so there
is a single configuration and the build is a handful of compiler invocations
that can run on a machine without a GPU (nvcc cross-compiles).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "lib"

HOST_SOURCES = [
    "host/allocator.cc",
    "host/team.cc",
    "host/runtime.cc",
    "host/cpu_backend.cc",
    "host/typed_api.cc",
    "host/proxy.cc",
    "host/unit_api.cc",
]

NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-std=c++17", "-O3", "-lineinfo", "--use_fast_math", "-Xcompiler", "-fPIC", "-shared",
              "--expt-relaxed-constexpr", "-Xptxas", "-v"]

# name -> (sources relative to csrc/, extra flags)
CUDA_TARGETS = {
    "libbshmem_cuda.so": (["cuda/vmm_heap.cu", "cuda/gpu_backend.cu", "cuda/coll_dispatch.cu", "cuda/coll_move.cu", "cuda/coll_reduce_f32.cu",
                           "cuda/coll_reduce_f16.cu", "cuda/coll_reduce_i32.cu", "cuda/coll_reduce_i8.cu", "cuda/p2p_kernels.cu", "cuda/api_matrix.cu", "cuda/functional_tester.cu", "cuda/functional_tester_coll.cu", "cuda/group_noalloc.cu", "cuda/gpu_proxy.cu", "cuda/device_util_kernels.cu"] + HOST_SOURCES, []),
    "libbshmem_gemm.so": (["cuda/gemm_bf16.cu"], []),
    "libbshmem_fused.so": (["cuda/fused_tp.cu"], []),
    "libbshmem_moe.so": (["cuda/moe_kernels.cu", "cuda/moe_gemm.cu"], []),
    "libbshmem_fp8.so": (["cuda/gemm_fp8.cu"], []),
}


def _nvcc() -> str | None:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if Path(cand).exists() else None


_INCLUDE_DIRS = [CSRC / "include", CSRC / "cuda", CSRC / "host"]


def _includes(src: Path, seen: set[Path]) -> None:
    """Transitive closure of the quoted #include files of `src` that live in this tree."""
    if src in seen or not src.exists():
        return
    seen.add(src)
    for line in src.read_text(errors="ignore").splitlines():
        line = line.strip()
        if line.startswith("#include \""):
            name = line.split("\"")[1]
            for d in [src.parent] + _INCLUDE_DIRS:
                if (d / name).exists():
                    _includes((d / name).resolve(), seen)
                    break


def _stale(out: Path, srcs: list[Path]) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    deps: set[Path] = set()
    for s in srcs:
        _includes(s.resolve(), deps)
    return any(d.stat().st_mtime > t for d in deps)


def _run(cmd: list[str], log: Path) -> None:
    p = subprocess.run(cmd, cwd=str(CSRC), capture_output=True, text=True)
    log.write_text("$ " + " ".join(cmd) + "\n" + p.stdout + p.stderr)
    if p.returncode != 0:
        raise RuntimeError(f"build failed: {' '.join(cmd)}\n{p.stdout}\n{p.stderr}")


def build_host(force: bool = False) -> Path:
    LIB.mkdir(exist_ok=True)
    out = LIB / "libbshmem_host.so"
    srcs = [CSRC / s for s in HOST_SOURCES if (CSRC / s).exists()]
    if force or _stale(out, srcs):
        cmd = ["g++", "-std=c++17", "-O2", "-g", "-fPIC", "-shared", "-Wall", "-Wextra", "-o", str(out)] + \
            [str(s) for s in srcs] + ["-lpthread", "-lrt", "-ldl"]
        _run(cmd, LIB / "libbshmem_host.build.log")
    return out


def build_sanitizer_driver(kind: str, force: bool = False) -> Path:
    """The host runtime and its native stress driver (csrc/host/sanitize_main.cc) as one executable built with
    -fsanitize=<kind> ("thread" or "address"): data races and memory errors in the allocator, the team table, the
    CPU backend and the reverse-offload ring show up when the driver runs (tests/test_host_sanitizers.py)."""
    if kind not in ("thread", "address"):
        raise ValueError("kind must be 'thread' or 'address'")
    LIB.mkdir(exist_ok=True)
    out = LIB / f"bshmem_sanitize_{kind}"
    srcs = [CSRC / s for s in HOST_SOURCES] + [CSRC / "host/sanitize_main.cc"]
    if force or _stale(out, srcs):
        cmd = ["g++", "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", f"-fsanitize={kind}", "-o", str(out)] + \
            [str(s) for s in srcs] + ["-lpthread", "-lrt", "-ldl"]
        _run(cmd, LIB / f"bshmem_sanitize_{kind}.build.log")
    return out


def _compile_object(nvcc: str, src: Path, obj: Path, extra: list[str], force: bool) -> str:
    if force or _stale(obj, [src]):
        flags = [f for f in NVCC_FLAGS if f != "-shared"]
        cmd = [nvcc] + NVCC_ARCH + flags + extra + ["-I", str(CSRC / "include"), "-I", str(CSRC / "cuda"), "-c", "-o", str(obj), str(src)]
        _run(cmd, obj.with_suffix(".log"))       # .cc files are compiled as host C++ by nvcc
    return obj.with_suffix(".log").read_text() if obj.with_suffix(".log").exists() else ""


def build_cuda_target(name: str, force: bool = False) -> Path | None:
    """One shared object per target; its sources are compiled to objects in parallel, then linked."""
    nvcc = _nvcc()
    if nvcc is None:
        return None
    LIB.mkdir(exist_ok=True)
    srcs_rel, extra = CUDA_TARGETS[name]
    srcs = [CSRC / s for s in srcs_rel]
    if not all(s.exists() for s in srcs if s.suffix == ".cu"):
        return None   # target not written yet
    srcs = [s for s in srcs if s.exists()]
    out = LIB / name
    if force or _stale(out, srcs):
        objdir = LIB / "obj" / name.replace(".so", "")
        objdir.mkdir(parents=True, exist_ok=True)
        objs = [objdir / (s.stem + ".o") for s in srcs]
        with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 2)) as ex:
            logs = list(ex.map(lambda so: _compile_object(nvcc, so[0], so[1], extra, force), zip(srcs, objs)))
        cmd = [nvcc] + NVCC_ARCH + ["-shared", "-o", str(out)] + [str(o) for o in objs] + ["-lpthread", "-lrt", "-ldl"]
        _run(cmd, LIB / (name + ".link.log"))
        (LIB / (name + ".build.log")).write_text("\n".join(logs))     # registers / spills / shared memory per kernel
    return out


def build_all(force: bool = False, cuda: bool = True) -> dict[str, str]:
    """Build everything that has sources; returns {artefact: path}."""
    built = {"libbshmem_host.so": str(build_host(force))}
    if cuda and _nvcc() is not None:
        with ThreadPoolExecutor(max_workers=min(6, os.cpu_count() or 2)) as ex:
            futs = {n: ex.submit(build_cuda_target, n, force) for n in CUDA_TARGETS}
            for n, f in futs.items():
                p = f.result()
                if p is not None:
                    built[n] = str(p)
    return built


def main() -> int:
    res = build_all(force="--force" in sys.argv)
    for k, v in res.items():
        print(f"{k}: {v}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
