"""Single-GPU GEMM benchmark: the tcgen05 kernel against cuBLAS (torch.matmul) on
the shapes of the tensor-parallel MLP, device-timed with CUDA events.

    python -m roc_shmem_b200.bench.gemm_bench [--iters 30] [--small]

Prints one JSON object per shape and a summary table; `--small` runs one small
problem once (used for profiler captures, where a launch is replayed many times).
"""
from __future__ import annotations

import argparse
import json

import torch

from ..ops.gemm import gemm_bf16, gemm_error_site

SHAPES = [
    ("down_proj_shard", 8192, 8192, 3584),
    ("gate_up_shard", 8192, 7168, 8192),
    ("square_8k", 8192, 8192, 8192),
    ("square_4k", 4096, 4096, 4096),
    ("moe_expert_up", 4096, 14336 * 2, 4096),
]


def time_fn(fn, iters: int, flush: torch.Tensor | None) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    total = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.zero_()            # 256 MiB write: evicts the 126 MB L2
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def run_fp8(args, dev) -> None:
    from ..ops.gemm_fp8 import fp8_error_site, gemm_fp8, quantize_act, quantize_weight
    if args.small:
        M, N, K = 2048, 2048, 2048
        qa = quantize_act(torch.randn(M, K, device=dev).to(torch.bfloat16))
        qw = quantize_weight((torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16))
        gemm_fp8(qa, qw)
        torch.cuda.synchronize()
        print(json.dumps({"small_fp8": [M, N, K], "error_site": fp8_error_site()}))
        return
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for name, M, N, K in SHAPES:
        a = torch.randn(M, K, device=dev).to(torch.bfloat16)
        b = (torch.randn(N, K, device=dev) * 0.02).to(torch.bfloat16)
        qa, qw = quantize_act(a), quantize_weight(b)
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        ref = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        ms_fp8 = time_fn(lambda: gemm_fp8(qa, qw, out, max_ctas=args.max_ctas), args.iters, flush)
        ms_quant = time_fn(lambda: quantize_act(a), args.iters, flush)
        ms_bf16 = time_fn(lambda: gemm_bf16(a, b, ref), args.iters, flush)
        exact = qa.dequantize() @ qw.dequantize().t()
        fl = 2.0 * M * N * K
        row = {"shape": name, "M": M, "N": N, "K": K, "ms_fp8": round(ms_fp8, 4), "ms_quant_act": round(ms_quant, 4),
               "ms_bf16_ours": round(ms_bf16, 4), "tflops_fp8": round(fl / ms_fp8 / 1e9, 1),
               "fp8_over_bf16": round(ms_bf16 / ms_fp8, 3),
               "max_abs_diff_vs_dequant_fp32": (out.float() - exact).abs().max().item(),
               "max_abs_diff_vs_bf16": (out.float() - ref.float()).abs().max().item(), "ref_scale": ref.float().abs().max().item(),
               "error_site": fp8_error_site()}
        print(json.dumps(row), flush=True)
        del a, b, qa, qw, out, ref, exact


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--mid", action="store_true", help="one launch of a 4-wave problem (592 tiles) for profiler captures")
    ap.add_argument("--max-ctas", type=int, default=0)
    ap.add_argument("--fp8", action="store_true", help="block-scaled fp8 kernel against the bf16 kernel and cuBLAS bf16")
    args = ap.parse_args()
    dev = torch.device("cuda")
    if args.fp8:
        run_fp8(args, dev)
        return
    if args.small or args.mid:
        M, N, K = (4096, 9472, 4096) if args.mid else (2048, 2048, 2048)
        a = torch.randn(M, K, device=dev).to(torch.bfloat16)
        b = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)
        pad = torch.empty(160 << 20, dtype=torch.uint8, device=dev)
        pad.zero_()
        out = gemm_bf16(a, b)
        torch.cuda.synchronize()
        print(json.dumps({"small": [M, N, K], "error_site": gemm_error_site()}))
        return
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows = []
    for name, M, N, K in SHAPES:
        a = torch.randn(M, K, device=dev).to(torch.bfloat16)
        b = (torch.randn(N, K, device=dev) * 0.02).to(torch.bfloat16)
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        ref = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        ms_ours = time_fn(lambda: gemm_bf16(a, b, out, max_ctas=args.max_ctas), args.iters, flush)
        ms_cublas = time_fn(lambda: torch.matmul(a, b.t(), out=ref), args.iters, flush)
        err = (out.float() - ref.float()).abs().max().item()
        fl = 2.0 * M * N * K
        row = {"shape": name, "M": M, "N": N, "K": K, "ms_ours": round(ms_ours, 4), "ms_cublas": round(ms_cublas, 4),
               "tflops_ours": round(fl / ms_ours / 1e9, 1), "tflops_cublas": round(fl / ms_cublas / 1e9, 1),
               "ours_over_cublas": round(ms_cublas / ms_ours, 3), "max_abs_diff_vs_cublas": err,
               "error_site": gemm_error_site()}
        rows.append(row)
        print(json.dumps(row), flush=True)
        del a, b, out, ref


if __name__ == "__main__":
    main()
