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
    "libbshmem_cuda.so": (["cuda/vmm_heap.cu", "cuda/gpu_backend.cu", "cuda/p2p_kernels.cu", "cuda/group_noalloc.cu", "cuda/gpu_proxy.cu", "cuda/device_util_kernels.cu"] + HOST_SOURCES, []),
    "libbshmem_gemm.so": (["cuda/gemm_bf16.cu"], []),
    "libbshmem_fused.so": (["cuda/fused_tp.cu"], []),
    "libbshmem_moe.so": (["cuda/moe_kernels.cu", "cuda/moe_gemm.cu"], []),
    "libbshmem_fp8.so": (["cuda/gemm_fp8.cu"], []),
}


def _nvcc() -> str | None:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if Path(cand).exists() else None


def _stale(out: Path, srcs: list[Path]) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    deps = list(srcs) + list((CSRC / "include").glob("*")) + list((CSRC / "host").glob("*.h")) + \
        list((CSRC / "cuda").glob("*.cuh"))
    return any(d.exists() and d.stat().st_mtime > t for d in deps)


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


def build_cuda_target(name: str, force: bool = False) -> Path | None:
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
        cmd = [nvcc] + NVCC_ARCH + NVCC_FLAGS + extra + ["-I", str(CSRC / "include"), "-I", str(CSRC / "cuda"),
                                                         "-o", str(out)] + [str(s) for s in srcs] + ["-lpthread", "-lrt", "-ldl"]
        # .cc files listed next to .cu ones are compiled as host C++ by nvcc.
        _run(cmd, LIB / (name + ".build.log"))
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


if __name__ == "__main__":
    res = build_all(force="--force" in sys.argv)
    for k, v in res.items():
        print(f"{k}: {v}")
