"""Fused tensor-parallel kernels: GEMM → reduce-scatter and all-gather → GEMM.

One hand-written sm_100a kernel per op does the tcgen05 GEMM *and* moves the tiles
over NVLink peer memory (TMA stores + signal words one way, peer loads + arrival
counters the other); see csrc/cuda/fused_tp.cu.  The NCCL + cuBLAS equivalents used
as the baseline are in roc_shmem_b200/baseline/tp.py.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _native
from ..gpu import DevState

_declared = False


def fused_lib() -> C.CDLL:
    global _declared
    lib = _native.load("libbshmem_fused.so")
    if not _declared:
        VP, I, U64 = C.c_void_p, C.c_int, C.c_uint64
        lib.bshmem_fused_last_error.restype = C.c_char_p
        lib.bshmem_fused_rs_staging_bytes.restype = U64
        lib.bshmem_fused_rs_staging_bytes.argtypes = [I, I]
        lib.bshmem_fused_rs_signal_bytes.restype = U64
        lib.bshmem_fused_rs_signal_bytes.argtypes = [I, I, I]
        lib.bshmem_fused_rs_plan.restype = I
        lib.bshmem_fused_rs_plan.argtypes = [C.POINTER(DevState), I, I, I, VP, VP, C.POINTER(VP)]
        lib.bshmem_fused_rs_run.restype = I
        lib.bshmem_fused_rs_run.argtypes = [VP, VP, I, VP, I, VP, I, VP, I, I]
        lib.bshmem_fused_ag_flag_bytes.restype = U64
        lib.bshmem_fused_ag_flag_bytes.argtypes = [I]
        lib.bshmem_fused_ag_plan.restype = I
        lib.bshmem_fused_ag_plan.argtypes = [C.POINTER(DevState), I, I, I, VP, VP, C.POINTER(VP)]
        lib.bshmem_fused_ag_run.restype = I
        lib.bshmem_fused_ag_run.argtypes = [VP, VP, I, VP, I, VP, I, I]
        lib.bshmem_fused_error_site.restype = I
        lib.bshmem_fused_error_site.argtypes = [VP, I]
        lib.bshmem_fused_destroy.restype = I
        lib.bshmem_fused_destroy.argtypes = [VP]
        _declared = True
    return lib


def _check(lib, st: int, what: str) -> None:
    if st != 0:
        raise RuntimeError(f"{what} failed ({st}): {lib.bshmem_fused_last_error().decode()}")


class GemmReduceScatter:
    """out[M/P, N] (this PE's rows) = sum over PEs r of x_r[M, K] @ w_r[N, K].T"""

    algorithm = ("one kernel: tcgen05 GEMM on CTA pairs (cta_group::2, 256x256 tiles, two TMEM accumulator stages) whose "
                 "epilogue TMA-stores bf16 partial tiles into the owner PE's staging over NVLink + one signal per CTA and "
                 "tile; a PE's own tiles come last and their epilogue adds the P-1 arrived partials to the fp32 accumulators")

    def __init__(self, rt, M: int, N: int, K: int, timeout_ms: int = 2000, max_ctas: int = 0):
        self.rt, self.M, self.N, self.K = rt, M, N, K
        self.lib = fused_lib()
        P = rt.n_pes
        self.timeout_ms, self.max_ctas = timeout_ms, max_ctas
        self.staging = rt.empty((self.lib.bshmem_fused_rs_staging_bytes(M, N),), torch.uint8, align=1024)
        nsig = self.lib.bshmem_fused_rs_signal_bytes(M, N, P) // 8
        self.signals = rt.zeros((nsig,), torch.int64)
        self.out = torch.empty((M // P, N), dtype=torch.bfloat16, device=rt.device)
        st = rt.device_state()
        plan = C.c_void_p()
        _check(self.lib, self.lib.bshmem_fused_rs_plan(C.byref(st), M, N, K, self.staging.data_ptr(),
                                                       self.signals.data_ptr(), C.byref(plan)), "gemm_rs plan")
        self.plan = plan
        rt.barrier_all()      # every PE's signal words are zero before anyone sends

    def __call__(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None) -> int:
        """Enqueue on the current stream; returns the number of kernels launched (1)."""
        out = self.out if out is None else out
        st = self.lib.bshmem_fused_rs_run(self.plan, x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(),
                                          out.stride(0), torch.cuda.current_stream().cuda_stream, self.timeout_ms,
                                          self.max_ctas)
        _check(self.lib, st, "gemm_rs run")
        return 1

    def check(self) -> None:
        site = self.lib.bshmem_fused_error_site(self.plan, 1)
        if site:
            raise RuntimeError(f"gemm_rs: a bounded in-kernel wait ran out (site {site})")

    def close(self) -> None:
        if self.plan:
            self.lib.bshmem_fused_destroy(self.plan)
            self.plan = None


class AllGatherGemm:
    """out[M, N] = gather_rows(x_shards)[M, K] @ w[N, K].T ; this PE's shard lives in ``self.x_shard``
    (a view into the symmetric gathered buffer), so writing activations there is the only input step."""

    algorithm = ("one kernel: tcgen05 GEMM whose epilogue warps pull the peers' activation rows over NVLink in "
                 "schedule order while the tensor core runs; TMA producers wait on per-256-row arrival counters")

    def __init__(self, rt, M: int, N: int, K: int, timeout_ms: int = 2000, max_ctas: int = 0):
        self.rt, self.M, self.N, self.K = rt, M, N, K
        self.lib = fused_lib()
        P = rt.n_pes
        self.timeout_ms, self.max_ctas = timeout_ms, max_ctas
        self.xg = rt.empty((M, K), torch.bfloat16, align=1024)
        rows = M // P
        self.x_shard = self.xg[rt.my_pe * rows:(rt.my_pe + 1) * rows]
        self.flags = rt.zeros((2 * P,), torch.int64)
        self.out = torch.empty((M, N), dtype=torch.bfloat16, device=rt.device)
        st = rt.device_state()
        plan = C.c_void_p()
        _check(self.lib, self.lib.bshmem_fused_ag_plan(C.byref(st), M, N, K, self.xg.data_ptr(), self.flags.data_ptr(),
                                                       C.byref(plan)), "ag_gemm plan")
        self.plan = plan
        rt.barrier_all()

    def __call__(self, w: torch.Tensor, out: torch.Tensor | None = None) -> int:
        out = self.out if out is None else out
        st = self.lib.bshmem_fused_ag_run(self.plan, w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0),
                                          torch.cuda.current_stream().cuda_stream, self.timeout_ms, self.max_ctas)
        _check(self.lib, st, "ag_gemm run")
        return 1

    def check(self) -> None:
        site = self.lib.bshmem_fused_error_site(self.plan, 1)
        if site:
            raise RuntimeError(f"ag_gemm: a bounded in-kernel wait ran out (site {site})")

    def close(self) -> None:
        if self.plan:
            self.lib.bshmem_fused_destroy(self.plan)
            self.plan = None
