"""Hand-written tcgen05 GEMM (sm_100a): ``C = A @ B.T`` with A [M, K], B [N, K].

This is the compute core under the fused tensor-parallel kernels; the reference
contains no GEMM (it is a communication runtime only), so there is no parity
citation — the layout convention is torch's ``F.linear(x, w)``.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from .. import _native

_declared = False


def gemm_lib() -> C.CDLL:
    global _declared
    lib = _native.load("libbshmem_gemm.so")
    if not _declared:
        lib.bshmem_gemm_last_error.restype = C.c_char_p
        lib.bshmem_gemm_bf16.restype = C.c_int
        lib.bshmem_gemm_bf16.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                         C.c_int, C.c_void_p, C.c_int, C.c_int]
        lib.bshmem_gemm_error_site.restype = C.c_int
        lib.bshmem_gemm_error_site.argtypes = [C.c_int]
        _declared = True
    return lib


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None, *, max_ctas: int = 0,
              timeout_ms: int = 2000) -> torch.Tensor:
    """out[M, N] = a[M, K] @ b[N, K].T in bf16 with fp32 accumulation (tcgen05 + TMEM).

    Launches on the current CUDA stream.  Fails loudly if the native library is
    missing — there is no eager fallback."""
    if not (a.is_cuda and b.is_cuda):
        raise ValueError("gemm_bf16 needs CUDA tensors")
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise ValueError("gemm_bf16 needs bf16 operands")
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[1]:
        raise ValueError(f"shape mismatch: a {tuple(a.shape)} b {tuple(b.shape)}")
    if a.stride(1) != 1 or b.stride(1) != 1:
        raise ValueError("operands must be K-major (last dimension contiguous)")
    M, K = a.shape
    N = b.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    elif out.shape != (M, N) or out.dtype != torch.bfloat16 or out.stride(1) != 1:
        raise ValueError("bad output tensor")
    lib = gemm_lib()
    st = lib.bshmem_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0),
                              out.stride(0), torch.cuda.current_stream().cuda_stream, max_ctas, timeout_ms)
    if st != 0:
        raise RuntimeError(f"bshmem_gemm_bf16 failed ({st}): {lib.bshmem_gemm_last_error().decode()}")
    return out


def gemm_error_site(clear: bool = True) -> int:
    """0 if no in-kernel bounded wait ran out since the last clear, else the site code."""
    return int(gemm_lib().bshmem_gemm_error_site(int(clear)))
