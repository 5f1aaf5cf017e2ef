"""Fused TP kernels vs NCCL + cuBLAS on the same buffers: correctness and device time.

    torchrun --nproc-per-node P -m roc_shmem_b200.bench.tp_bench [--small] [--iters 20] [--out file.json]

Config: Llama-3-70B MLP, tokens M = 8192, hidden 8192, ffn 28672 split over P ranks
(K/rank = 28672/P for the down projection, N/rank = 2*28672/P for gate+up), bf16,
activations N(0,1), weights N(0,0.02).  `--small` shrinks everything for tests.
Timing: CUDA events per rank, max over ranks; roofline = max(FLOPs / measured GEMM
peak, NVLink bytes / 770 GB/s).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

import roc_shmem_b200 as shmem
from roc_shmem_b200.baseline import tp as base
from roc_shmem_b200.ops.fused_tp import AllGatherGemm, GemmReduceScatter


def timed(fn, iters: int, rt) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    rt.barrier_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    t = torch.tensor([ms], device="cuda")
    if dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--mid", action="store_true", help="4096-token, hidden 4096, ffn 4096*P problem (profiler captures)")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--out", default="")
    ap.add_argument("--peak-tflops", type=float, default=1399.1)
    ap.add_argument("--link-gbs", type=float, default=770.0)
    args = ap.parse_args()
    for k, v in (("RANK", "0"), ("WORLD_SIZE", "1"), ("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", "29535")):
        os.environ.setdefault(k, v)                        # plain `python -m ...` = one rank
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rt = shmem.init("device", device=local, heap_bytes=(256 << 20) if args.small else (3 << 30))
    dev = torch.device("cuda", local)
    P = world
    if args.small:
        M, H, F = 512 * P, 512, 256 * P
    elif args.mid:
        M, H, F = 4096, 4096, 4096 * P
    else:
        M, H, F = 8192, 8192, 28672
    results = {"world": P, "M": M, "hidden": H, "ffn": F}
    torch.manual_seed(100 + rank)

    # ---------------- GEMM -> reduce-scatter (down projection) ----------------
    K = F // P
    x = torch.randn(M, K, device=dev).to(torch.bfloat16)
    w = (torch.randn(H, K, device=dev) * 0.02).to(torch.bfloat16)
    fused = GemmReduceScatter(rt, M, H, K)
    partial = torch.empty(M, H, device=dev, dtype=torch.bfloat16)
    ref = torch.empty(M // P, H, device=dev, dtype=torch.bfloat16)
    fused(x, w)
    base.gemm_reduce_scatter(x, w, partial, ref)
    torch.cuda.synchronize()
    fused.check()
    diff = (fused.out.float() - ref.float()).abs().max().item()
    scale = ref.float().abs().max().item()
    results["rs_max_abs_diff"] = diff
    results["rs_ref_scale"] = scale
    ok_rs = diff <= 2e-2 * scale + 1e-3
    ms_f = timed(lambda: fused(x, w), args.iters, rt)
    ms_b = timed(lambda: base.gemm_reduce_scatter(x, w, partial, ref), args.iters, rt)
    fused.check()
    flops = 2.0 * M * H * K
    link_bytes = (P - 1) / P * M * H * 2
    roof_ms = max(flops / (args.peak_tflops * 1e12), link_bytes / (args.link_gbs * 1e9)) * 1e3
    results.update({"rs_ms_fused": ms_f, "rs_ms_nccl_cublas": ms_b, "rs_speedup": ms_b / ms_f, "rs_roofline_ms": roof_ms,
                    "rs_roofline_frac": roof_ms / ms_f, "rs_ok": bool(ok_rs)})
    fused.close()
    del partial, ref, x, w

    # ---------------- all-gather -> GEMM (gate + up projection) ----------------
    N = 2 * F // P
    ag = AllGatherGemm(rt, M, N, H)
    ag.x_shard.copy_(torch.randn(M // P, H, device=dev).to(torch.bfloat16))
    w2 = (torch.randn(N, H, device=dev) * 0.02).to(torch.bfloat16)
    gathered = torch.empty(M, H, device=dev, dtype=torch.bfloat16)
    ref2 = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    rt.barrier_all()
    ag(w2)
    base.all_gather_gemm(ag.x_shard, w2, gathered, ref2)
    torch.cuda.synchronize()
    ag.check()
    diff2 = (ag.out.float() - ref2.float()).abs().max().item()
    scale2 = ref2.float().abs().max().item()
    gather_exact = bool(torch.equal(ag.xg, gathered))
    results.update({"ag_max_abs_diff": diff2, "ag_ref_scale": scale2, "ag_gather_exact": gather_exact})
    ok_ag = diff2 <= 2e-2 * scale2 + 1e-3 and gather_exact
    ms_f2 = timed(lambda: ag(w2), args.iters, rt)
    ms_b2 = timed(lambda: base.all_gather_gemm(ag.x_shard, w2, gathered, ref2), args.iters, rt)
    ag.check()
    flops2 = 2.0 * M * N * H
    link2 = (P - 1) / P * M * H * 2
    roof2 = max(flops2 / (args.peak_tflops * 1e12), link2 / (args.link_gbs * 1e9)) * 1e3
    results.update({"ag_ms_fused": ms_f2, "ag_ms_nccl_cublas": ms_b2, "ag_speedup": ms_b2 / ms_f2, "ag_roofline_ms": roof2,
                    "ag_roofline_frac": roof2 / ms_f2, "ag_ok": bool(ok_ag)})
    x_shard_bf16 = ag.x_shard.clone()
    ag.close()

    # ---------------- all-gather -> GEMM on block-scaled fp8 (e4m3 rows cross NVLink: half the bytes) ----------------
    from roc_shmem_b200.ops.gemm_fp8 import AllGatherGemmFp8, gemm_fp8, quantize_act, quantize_weight
    ok_ag8 = True
    if N % 256 == 0 and H % 128 == 0 and (M // P) % 128 == 0:
        ag8 = AllGatherGemmFp8(rt, M, N, H)
        qw = quantize_weight(w2)
        ag8.set_input(x_shard_bf16)
        rt.barrier_all()
        ag8(qw)
        dist.all_gather_into_tensor(gathered, x_shard_bf16)
        qa_full = quantize_act(gathered)                          # same quantiser on the same rows: identical operands
        ref8 = gemm_fp8(qa_full, qw)
        torch.cuda.synchronize()
        ag8.check()
        diff8 = (ag8.out.float() - ref8.float()).abs().max().item()
        gather8_exact = bool(torch.equal(ag8.xq, qa_full.q) and torch.equal(ag8.sa, qa_full.scales))
        ok_ag8 = diff8 == 0.0 and gather8_exact

        def step8():
            ag8.set_input(x_shard_bf16)                           # the quantisation of the local rows is part of the step
            ag8(qw)
        ms_f8 = timed(step8, args.iters, rt)
        ag8.check()
        results.update({"ag_fp8_max_abs_diff_vs_unfused_fp8": diff8, "ag_fp8_gather_exact": gather8_exact, "ag_fp8_ms_fused": ms_f8,
                        "ag_fp8_speedup_vs_bf16_nccl_cublas": ms_b2 / ms_f8, "ag_fp8_speedup_vs_bf16_fused": ms_f2 / ms_f8,
                        "ag_fp8_vs_bf16_max_abs_diff": (ag8.out.float() - ref2.float()).abs().max().item(), "ag_fp8_ok": bool(ok_ag8)})
        ag8.close()

    # ---------------- GEMM -> reduce-scatter on block-scaled fp8 operands ----------------
    from roc_shmem_b200.ops.gemm_fp8 import GemmReduceScatterFp8
    ok_rs8 = True
    if H % 256 == 0 and K % 128 == 0 and (M // P) % 128 == 0:
        torch.manual_seed(300 + rank)
        x8 = torch.randn(M, K, device=dev).to(torch.bfloat16)
        w8 = (torch.randn(H, K, device=dev) * 0.02).to(torch.bfloat16)
        qx, qwd = quantize_act(x8), quantize_weight(w8)
        rs8 = GemmReduceScatterFp8(rt, M, H, K)
        rs8(qx, qwd)
        part = gemm_fp8(qx, qwd).float()                          # this rank's bf16-rounded partial, summed in fp32 by NCCL
        ref_rs8 = torch.empty(M // P, H, device=dev, dtype=torch.float32)
        dist.reduce_scatter_tensor(ref_rs8, part)
        torch.cuda.synchronize()
        rs8.check()
        diff_rs8 = (rs8.out.float() - ref_rs8).abs().max().item()
        scale_rs8 = ref_rs8.abs().max().item()
        ok_rs8 = diff_rs8 <= 1e-2 * scale_rs8 + 1e-3               # one bf16 rounding of the fp32 sum
        ms_rs8 = timed(lambda: rs8(qx, qwd), args.iters, rt)
        rs8.check()
        results.update({"rs_fp8_max_abs_diff": diff_rs8, "rs_fp8_ref_scale": scale_rs8, "rs_fp8_ms_fused": ms_rs8,
                        "rs_fp8_speedup_vs_bf16_nccl_cublas": results["rs_ms_nccl_cublas"] / ms_rs8,
                        "rs_fp8_speedup_vs_bf16_fused": results["rs_ms_fused"] / ms_rs8, "rs_fp8_ok": bool(ok_rs8)})
        rs8.close()
        del x8, w8, part

    oks = torch.tensor([int(ok_rs and ok_ag and ok_ag8 and ok_rs8)], device=dev)
    dist.all_reduce(oks, op=dist.ReduceOp.MIN)
    results["all_ranks_ok"] = bool(oks.item())
    if rank == 0:
        line = json.dumps(results)
        print(line, flush=True)
        if args.out:
            os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
            with open(args.out, "w") as f:
                f.write(line + "\n")
    shmem.finalize()
    dist.destroy_process_group()
    if not results["all_ranks_ok"]:
        raise SystemExit(1)


if __name__ == "__main__":
    main()
