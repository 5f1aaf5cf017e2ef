"""Tensor-parallel Llama MLP block (forward, forward+backward) against NCCL + cuBLAS doing the same
sharded math: all_gather → matmul → SwiGLU → matmul → reduce_scatter and the matching backward.

    torchrun --nproc-per-node P -m roc_shmem_b200.bench.mlp_bench [--small] [--iters 10] [--out file.json]

Config: Llama-3-70B MLP (hidden 8192, FFN 28672 split over P ranks), 8192 tokens, bf16, activations N(0,1),
weights N(0,0.02).  Device-timed with CUDA events, max over ranks.  One step touches > 1 GB per rank, far more
than the 126 MB L2, so no explicit flush is needed.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist
import torch.nn.functional as Fnn

import roc_shmem_b200 as shmem
from roc_shmem_b200.models.llama import LlamaMLP


class NcclMLP:
    """The baseline: NCCL collectives + cuBLAS GEMMs + eager SwiGLU on the same shards (hand-written backward,
    same set of GEMMs as the fused block)."""

    def __init__(self, wg, wu, wd, M: int, P: int):
        self.wg, self.wu, self.wd, self.M, self.P = wg, wu, wd, M, P
        H = wg.shape[1]
        self.w13 = torch.cat((wg, wu))                        # [2Fp, H]
        self.xg = torch.empty((M, H), dtype=torch.bfloat16, device=wg.device)
        self.dyg = torch.empty((M, H), dtype=torch.bfloat16, device=wg.device)
        self.y = torch.empty((M // P, H), dtype=torch.bfloat16, device=wg.device)
        self.dx = torch.empty((M // P, H), dtype=torch.bfloat16, device=wg.device)

    def forward(self, x_shard):
        if self.P > 1:
            dist.all_gather_into_tensor(self.xg, x_shard)
        else:
            self.xg.copy_(x_shard)
        self.gu = self.xg @ self.w13.t()
        Fp = self.wg.shape[0]
        self.g, self.u = self.gu[:, :Fp], self.gu[:, Fp:]
        self.h = Fnn.silu(self.g) * self.u
        part = self.h @ self.wd.t()
        if self.P > 1:
            dist.reduce_scatter_tensor(self.y, part)
        else:
            self.y = part
        return self.y

    def backward(self, dy_shard):
        if self.P > 1:
            dist.all_gather_into_tensor(self.dyg, dy_shard)
        else:
            self.dyg.copy_(dy_shard)
        dh = self.dyg @ self.wd
        self.dwd = self.dyg.t() @ self.h
        sg = torch.sigmoid(self.g.float())
        dg = (dh.float() * self.u.float() * sg * (1 + self.g.float() * (1 - sg))).to(torch.bfloat16)
        du = (dh.float() * (self.g.float() * sg)).to(torch.bfloat16)
        dgu = torch.cat((dg, du), dim=1)
        self.dw13 = dgu.t() @ self.xg
        part = dgu @ self.w13
        if self.P > 1:
            dist.reduce_scatter_tensor(self.dx, part)
        else:
            self.dx = part
        return self.dx


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
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    if dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    for k, v in (("RANK", "0"), ("WORLD_SIZE", "1"), ("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", "29534")):
        os.environ.setdefault(k, v)                        # plain `python -m ...` = one rank
    rank, P = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if args.small:
        M, H, F = 512 * P, 512, 512 * P
    else:
        M, H, F = 8192, 8192, 28672
    Fp = F // P
    rt = shmem.init("device", device=local, heap_bytes=(512 << 20) if args.small else (2 << 30), timeout_ms=20000)
    dev = rt.device
    torch.manual_seed(100 + rank)
    wg = (torch.randn(Fp, H, device=dev) * 0.02).to(torch.bfloat16)
    wu = (torch.randn(Fp, H, device=dev) * 0.02).to(torch.bfloat16)
    wd = (torch.randn(H, Fp, device=dev) * 0.02).to(torch.bfloat16)
    x = torch.randn(M // P, H, device=dev).to(torch.bfloat16)
    dy = torch.randn(M // P, H, device=dev).to(torch.bfloat16)
    block = LlamaMLP(rt, H, F, M)
    block.load(wg, wu, wd)
    rt.set_blocking(False)
    base = NcclMLP(wg, wu, wd, M, P)

    y = block.forward(x).clone()
    dx = block.backward(dy).clone()
    yb = base.forward(x).clone()
    dxb = base.backward(dy).clone()
    torch.cuda.synchronize()
    block.check()
    res = {"world": P, "tokens": M, "hidden": H, "ffn": F,
           "fwd_max_abs_diff": (y.float() - yb.float()).abs().max().item(), "fwd_scale": yb.float().abs().max().item(),
           "dx_max_abs_diff": (dx.float() - dxb.float()).abs().max().item(), "dx_scale": dxb.float().abs().max().item(),
           "dw2_rel_diff": ((block.dw2.float() - base.dwd.float()).abs().max() / base.dwd.float().abs().max()).item()}
    ok = res["fwd_max_abs_diff"] <= 0.03 * res["fwd_scale"] + 0.02 and res["dx_max_abs_diff"] <= 0.03 * res["dx_scale"] + 0.02 \
        and res["dw2_rel_diff"] < 0.03

    def ours_fb():
        block.forward(x)
        block.backward(dy)

    def base_fb():
        base.forward(x)
        base.backward(dy)

    res["ms_fwd"] = timed(lambda: block.forward(x), args.iters, rt)
    res["ms_fwd_bwd"] = timed(ours_fb, args.iters, rt)
    res["ms_fwd_nccl_cublas"] = timed(lambda: base.forward(x), args.iters, rt)
    res["ms_fwd_bwd_nccl_cublas"] = timed(base_fb, args.iters, rt)
    flops_fwd = 2.0 * M * H * (3 * Fp)                         # per rank: gate+up (2Fp) and down (Fp)
    res["tflops_fwd_per_gpu"] = flops_fwd / res["ms_fwd"] / 1e9
    res["tflops_fwd_bwd_per_gpu"] = 3 * flops_fwd / res["ms_fwd_bwd"] / 1e9
    res["speedup_fwd"] = res["ms_fwd_nccl_cublas"] / res["ms_fwd"]
    res["speedup_fwd_bwd"] = res["ms_fwd_bwd_nccl_cublas"] / res["ms_fwd_bwd"]
    torch.cuda.synchronize()
    block.check()
    flag = torch.tensor([1 if ok else 0], device=dev)
    if P > 1:
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    res["all_ranks_ok"] = bool(flag.item())
    if rank == 0:
        print(json.dumps(res), flush=True)
        if args.out:
            with open(args.out, "w") as f:
                json.dump(res, f)
    rt.barrier_all()
    shmem.finalize()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
