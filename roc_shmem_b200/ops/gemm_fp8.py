"""Block-scaled fp8 (e4m3) GEMM on the tcgen05 tensor cores, with its quantisers.

Scaling follows the fine-grained recipe used for fp8 training: activations carry one fp32
scale per row and 128 columns (stored ``[K/128, M]`` so a warp's rows are contiguous),
weights one per 128x128 block (``[K/128, N/128]``).  The reference is a communication runtime
and contains no GEMM, so there is no parity citation.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from .. import _native

_declared = False


def fp8_lib() -> C.CDLL:
    global _declared
    lib = _native.load("libbshmem_fp8.so")
    if not _declared:
        VP, I = C.c_void_p, C.c_int
        lib.bshmem_fp8_last_error.restype = C.c_char_p
        lib.bshmem_gemm_fp8_blockscale.restype = I
        lib.bshmem_gemm_fp8_blockscale.argtypes = [VP, VP, VP, VP, VP, I, I, I, I, VP, I, I]
        lib.bshmem_fp8_quant_act.restype = I
        lib.bshmem_fp8_quant_act.argtypes = [VP, I, I, I, VP, VP, VP]
        lib.bshmem_fp8_quant_weight.restype = I
        lib.bshmem_fp8_quant_weight.argtypes = [VP, I, I, I, VP, VP, VP]
        lib.bshmem_fp8_error_site.restype = I
        lib.bshmem_fp8_error_site.argtypes = [I]
        lib.bshmem_fp8_quant_act_ld.restype = I
        lib.bshmem_fp8_quant_act_ld.argtypes = [VP, I, I, I, VP, VP, I, VP]
        lib.bshmem_fp8_ag_flag_bytes.restype = C.c_uint64
        lib.bshmem_fp8_ag_flag_bytes.argtypes = [I]
        lib.bshmem_fp8_ag_plan.restype = I
        lib.bshmem_fp8_ag_plan.argtypes = [VP, I, I, I, VP, VP, VP, C.POINTER(VP)]
        lib.bshmem_fp8_ag_run.restype = I
        lib.bshmem_fp8_ag_run.argtypes = [VP, VP, VP, VP, I, VP, I, I]
        lib.bshmem_fp8_ag_error_site.restype = I
        lib.bshmem_fp8_ag_error_site.argtypes = [VP, I]
        lib.bshmem_fp8_ag_destroy.restype = I
        lib.bshmem_fp8_ag_destroy.argtypes = [VP]
        lib.bshmem_fp8_rs_staging_bytes.restype = C.c_uint64
        lib.bshmem_fp8_rs_staging_bytes.argtypes = [I, I]
        lib.bshmem_fp8_rs_signal_bytes.restype = C.c_uint64
        lib.bshmem_fp8_rs_signal_bytes.argtypes = [I, I, I]
        lib.bshmem_fp8_rs_plan.restype = I
        lib.bshmem_fp8_rs_plan.argtypes = [VP, I, I, I, VP, VP, C.POINTER(VP)]
        lib.bshmem_fp8_rs_run.restype = I
        lib.bshmem_fp8_rs_run.argtypes = [VP, VP, VP, VP, VP, VP, I, VP, I, I]
        lib.bshmem_fp8_rs_error_site.restype = I
        lib.bshmem_fp8_rs_error_site.argtypes = [VP, I]
        lib.bshmem_fp8_rs_destroy.restype = I
        lib.bshmem_fp8_rs_destroy.argtypes = [VP]
        _declared = True
    return lib


@dataclass
class Fp8Tensor:
    """e4m3 payload ``q`` (uint8 view, [rows, K]) and its fp32 block scales."""
    q: torch.Tensor
    scales: torch.Tensor
    kind: str               # "act" (1x128 blocks, scales [K/128, rows]) or "weight" (128x128, scales [K/128, rows/128])

    def dequantize(self) -> torch.Tensor:
        """fp32 reconstruction (for tests and reference computations)."""
        rows, K = self.q.shape
        x = self.q.view(torch.float8_e4m3fn).float().view(rows, K // 128, 128)
        if self.kind == "act":
            s = self.scales.t().contiguous().view(rows, K // 128, 1)
        else:
            s = self.scales.t().contiguous().repeat_interleave(128, dim=0).view(rows, K // 128, 1)
        return (x * s).view(rows, K)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def quantize_act(x: torch.Tensor) -> Fp8Tensor:
    """bf16 [M, K] (K % 128 == 0) → e4m3 with one scale per row and 128 columns."""
    if x.dtype != torch.bfloat16 or x.dim() != 2 or x.stride(1) != 1 or x.shape[1] % 128:
        raise ValueError("quantize_act needs a K-major bf16 matrix with K % 128 == 0")
    M, K = x.shape
    q = torch.empty((M, K), dtype=torch.uint8, device=x.device)
    s = torch.empty((K // 128, M), dtype=torch.float32, device=x.device)
    lib = fp8_lib()
    st = lib.bshmem_fp8_quant_act(x.data_ptr(), M, K, x.stride(0), q.data_ptr(), s.data_ptr(), _stream())
    if st != 0:
        raise RuntimeError(f"fp8 quantize_act failed ({st}): {lib.bshmem_fp8_last_error().decode()}")
    return Fp8Tensor(q, s, "act")


def quantize_weight(w: torch.Tensor) -> Fp8Tensor:
    """bf16 [N, K] (N, K % 128 == 0) → e4m3 with one scale per 128x128 block."""
    if w.dtype != torch.bfloat16 or w.dim() != 2 or w.stride(1) != 1 or w.shape[1] % 128 or w.shape[0] % 128:
        raise ValueError("quantize_weight needs a K-major bf16 matrix with N % 128 == 0 and K % 128 == 0")
    N, K = w.shape
    q = torch.empty((N, K), dtype=torch.uint8, device=w.device)
    s = torch.empty((K // 128, N // 128), dtype=torch.float32, device=w.device)
    lib = fp8_lib()
    st = lib.bshmem_fp8_quant_weight(w.data_ptr(), N, K, w.stride(0), q.data_ptr(), s.data_ptr(), _stream())
    if st != 0:
        raise RuntimeError(f"fp8 quantize_weight failed ({st}): {lib.bshmem_fp8_last_error().decode()}")
    return Fp8Tensor(q, s, "weight")


def gemm_fp8(a: Fp8Tensor, b: Fp8Tensor, out: Optional[torch.Tensor] = None, *, max_ctas: int = 0,
             timeout_ms: int = 2000) -> torch.Tensor:
    """out[M, N] (bf16) = dequant(a)[M, K] @ dequant(b)[N, K].T, scales applied per 128-wide k-block
    to fp32 partial products.  M % 128 == 0, N % 256 == 0, K % 128 == 0.  Current CUDA stream."""
    if a.kind != "act" or b.kind != "weight":
        raise ValueError("gemm_fp8 takes (activation, weight)")
    M, K = a.q.shape
    N = b.q.shape[0]
    if b.q.shape[1] != K:
        raise ValueError("K mismatch")
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.q.device)
    elif out.shape != (M, N) or out.dtype != torch.bfloat16 or out.stride(1) != 1:
        raise ValueError("bad output tensor")
    lib = fp8_lib()
    st = lib.bshmem_gemm_fp8_blockscale(a.q.data_ptr(), a.scales.data_ptr(), b.q.data_ptr(), b.scales.data_ptr(), out.data_ptr(),
                                        M, N, K, out.stride(0), _stream(), max_ctas, timeout_ms)
    if st != 0:
        raise RuntimeError(f"fp8 gemm failed ({st}): {lib.bshmem_fp8_last_error().decode()}")
    return out


def fp8_error_site(clear: bool = True) -> int:
    """0 if no in-kernel bounded wait ran out since the last clear, else the site code."""
    return int(fp8_lib().bshmem_fp8_error_site(int(clear)))


class AllGatherGemmFp8:
    """out[M, N] (bf16) = all_gather_rows(quantised activations)[M, K] @ dequant(weight)[N, K].T in ONE kernel:
    the block-scaled fp8 GEMM whose two extra warps per CTA pull the peers' e4m3 rows and scale columns over
    NVLink while the tensor core works on rows that have already arrived.  Gathering e4m3 instead of bf16 halves
    the bytes on the wire.  ``set_input(x_shard)`` quantises this PE's [M/P, K] bf16 rows into its slice of the
    symmetric buffers; ``__call__(weight)`` runs the kernel on the current stream."""

    algorithm = ("one kernel: block-scaled fp8 tcgen05 GEMM (128x256 tiles, per-k-block promotion) + 2 pull warps per CTA "
                 "fetching the peers' e4m3 rows and scales over NVLink; producers wait on per-128-row arrival counters")

    def __init__(self, rt, M: int, N: int, K: int, timeout_ms: int = 2000, max_ctas: int = 0):
        self.rt, self.M, self.N, self.K = rt, M, N, K
        self.lib = fp8_lib()
        P = rt.n_pes
        self.timeout_ms, self.max_ctas = timeout_ms, max_ctas
        self.xq = rt.empty((M, K), torch.uint8, align=1024)
        self.sa = rt.empty((K // 128, M), torch.float32, align=1024)
        self.flags = rt.zeros((2 * P,), torch.int64)
        self.rows = M // P
        self.row0 = rt.my_pe * self.rows
        self.out = torch.empty((M, N), dtype=torch.bfloat16, device=rt.device)
        st = rt.device_state()
        plan = C.c_void_p()
        rc = self.lib.bshmem_fp8_ag_plan(C.byref(st), M, N, K, self.xq.data_ptr(), self.sa.data_ptr(), self.flags.data_ptr(),
                                         C.byref(plan))
        if rc != 0:
            raise RuntimeError(f"ag_gemm_fp8 plan failed ({rc}): {self.lib.bshmem_fp8_last_error().decode()}")
        self.plan = plan
        rt.barrier_all()      # every PE's flag words are zero before anyone signals

    def set_input(self, x_shard: torch.Tensor) -> None:
        """Quantise this PE's rows (bf16 [M/P, K]) into its slice of the gathered e4m3 buffer and scale matrix."""
        if x_shard.shape != (self.rows, self.K) or x_shard.dtype != torch.bfloat16 or x_shard.stride(1) != 1:
            raise ValueError("set_input needs this PE's [M/P, K] bf16 rows")
        q = self.xq[self.row0:self.row0 + self.rows]
        rc = self.lib.bshmem_fp8_quant_act_ld(x_shard.data_ptr(), self.rows, self.K, x_shard.stride(0), q.data_ptr(),
                                              self.sa.data_ptr() + 4 * self.row0, self.M, _stream())
        if rc != 0:
            raise RuntimeError(f"fp8 quantise failed ({rc}): {self.lib.bshmem_fp8_last_error().decode()}")

    def __call__(self, weight: Fp8Tensor, out: Optional[torch.Tensor] = None) -> int:
        out = self.out if out is None else out
        rc = self.lib.bshmem_fp8_ag_run(self.plan, weight.q.data_ptr(), weight.scales.data_ptr(), out.data_ptr(), out.stride(0),
                                        _stream(), self.timeout_ms, self.max_ctas)
        if rc != 0:
            raise RuntimeError(f"ag_gemm_fp8 run failed ({rc}): {self.lib.bshmem_fp8_last_error().decode()}")
        return 1

    def gathered(self) -> Fp8Tensor:
        """The local gathered copy (complete after a call)."""
        return Fp8Tensor(self.xq, self.sa, "act")

    def check(self) -> None:
        site = self.lib.bshmem_fp8_ag_error_site(self.plan, 1)
        if site:
            raise RuntimeError(f"ag_gemm_fp8: a bounded in-kernel wait ran out (site {site})")

    def close(self) -> None:
        if self.plan:
            self.lib.bshmem_fp8_ag_destroy(self.plan)
            self.plan = None


class GemmReduceScatterFp8:
    """out[M/P, N] (this PE's rows, bf16) = sum over PEs r of dequant(a_r)[M, K] @ dequant(b_r)[N, K].T in ONE kernel:
    the block-scaled fp8 GEMM whose epilogue TMA-stores its bf16 partial tiles into the owner PE's staging over NVLink
    and signals per tile; after its last tile every CTA sums the P partials of the owned tiles dealt to it (fixed
    order, reproducible).  Staging is double-buffered by call parity and signals are monotonic, so back-to-back calls
    need no barrier."""

    algorithm = ("one kernel: block-scaled fp8 tcgen05 GEMM (128x256 tiles) whose epilogue TMA-stores bf16 partial tiles into "
                 "the owner PE's staging over NVLink + per-tile signal; CTAs then reduce the P partials of the owned tiles")

    def __init__(self, rt, M: int, N: int, K: int, timeout_ms: int = 2000, max_ctas: int = 0):
        self.rt, self.M, self.N, self.K = rt, M, N, K
        self.lib = fp8_lib()
        lib = self.lib
        P = rt.n_pes
        self.timeout_ms, self.max_ctas = timeout_ms, max_ctas
        self.staging = rt.empty((lib.bshmem_fp8_rs_staging_bytes(M, N),), torch.uint8, align=1024)
        self.signals = rt.zeros((max(1, lib.bshmem_fp8_rs_signal_bytes(M, N, P) // 8),), torch.int64)
        self.out = torch.empty((M // P, N), dtype=torch.bfloat16, device=rt.device)
        st = rt.device_state()
        plan = C.c_void_p()
        rc = lib.bshmem_fp8_rs_plan(C.byref(st), M, N, K, self.staging.data_ptr(), self.signals.data_ptr(), C.byref(plan))
        if rc != 0:
            raise RuntimeError(f"gemm_rs_fp8 plan failed ({rc}): {lib.bshmem_fp8_last_error().decode()}")
        self.plan = plan
        rt.barrier_all()      # every PE's signal words are zero before anyone sends

    def __call__(self, a: Fp8Tensor, b: Fp8Tensor, out: Optional[torch.Tensor] = None) -> int:
        if a.kind != "act" or b.kind != "weight" or a.q.shape != (self.M, self.K) or b.q.shape != (self.N, self.K):
            raise ValueError("gemm_rs_fp8 takes (activation [M, K], weight [N, K]) of the planned shape")
        out = self.out if out is None else out
        rc = self.lib.bshmem_fp8_rs_run(self.plan, a.q.data_ptr(), a.scales.data_ptr(), b.q.data_ptr(), b.scales.data_ptr(),
                                        out.data_ptr(), out.stride(0), _stream(), self.timeout_ms, self.max_ctas)
        if rc != 0:
            raise RuntimeError(f"gemm_rs_fp8 run failed ({rc}): {self.lib.bshmem_fp8_last_error().decode()}")
        return 1

    def check(self) -> None:
        site = self.lib.bshmem_fp8_rs_error_site(self.plan, 1)
        if site:
            raise RuntimeError(f"gemm_rs_fp8: a bounded in-kernel wait ran out (site {site})")

    def close(self) -> None:
        if self.plan:
            self.lib.bshmem_fp8_rs_destroy(self.plan)
            self.plan = None
