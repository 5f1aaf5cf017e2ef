"""Device collectives vs NCCL on identical buffers, teams of 2/4/8 PEs.

    torchrun --nproc-per-node P -m roc_shmem_b200.bench.coll_bench [--max-bytes 1073741824] [--out file.json]

Per-PE buffers 1 KiB .. max-bytes filled with N(0,1) (seed = PE); barrier, sum / max
allreduce and reduce-scatter in fp32 and bf16, fcollect and alltoall.  Results are
checked against NCCL's (bitwise for data movement; to rounding for reductions) and
both are device-timed with CUDA events, max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

import roc_shmem_b200 as shmem


def timed(fn, iters, rt):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    rt.barrier_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) * 1e3 / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def timed_graph(fn, iters, rt):
    """Same loop captured once in a CUDA graph and replayed: device time without the per-call host cost."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        rt.set_stream(side)                      # the runtime enqueues where it is told to
        for _ in range(2):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    rt.set_stream(torch.cuda.current_stream())
    rt.barrier_all()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        rt.set_stream(torch.cuda.current_stream())   # the capturing stream
        for _ in range(iters):
            fn()
    rt.set_stream(torch.cuda.current_stream())
    torch.cuda.synchronize()
    rt.barrier_all()
    g.replay()                                   # warm-up replay
    torch.cuda.synchronize()
    rt.barrier_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) * 1e3 / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--out", default="")
    ap.add_argument("--ctas", type=int, default=128)
    ap.add_argument("--nvls", action="store_true")
    ap.add_argument("--graph", action="store_true", help="also time barrier and small allreduces replayed from a CUDA graph")
    ap.add_argument("--team-sizes", default="", help="comma list: also time allreduce / fcollect on disjoint teams of that many PEs")
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    P = dist.get_world_size()
    # the heap's allocator hands out power-of-two blocks: source + destination + the runtime's own region
    rt = shmem.init("device", device=local, heap_bytes=4 * args.max_bytes + (512 << 20),
                    nvls="on" if args.nvls else "off", coll_ctas=args.ctas)
    me = rt.my_pe
    dev = rt.device
    rt.set_blocking(False)          # stream-ordered: calls enqueue kernels like NCCL does
    rows = []
    failed = []                      # every failed check of this rank: {"pe", "op", "bytes"}
    ok_all = True
    torch.manual_seed(me)

    # barrier latency
    us = timed(lambda: rt.barrier_all(), 50, rt)
    us_n = timed(lambda: dist.barrier(), 20, rt)
    rows.append({"op": "barrier", "bytes": 0, "us": us, "nccl_us": us_n})

    size = 1024
    sizes = []
    while size <= args.max_bytes:
        sizes.append(size)
        size *= 4
    if sizes[-1] != args.max_bytes:
        sizes.append(args.max_bytes)
    src_all = rt.empty((args.max_bytes,), torch.uint8, align=1024)
    dst_all = rt.empty((args.max_bytes,), torch.uint8, align=1024)
    for dtype in (torch.float32, torch.bfloat16):
        es = 2 if dtype == torch.bfloat16 else 4
        for nbytes in sizes:
            n = nbytes // es
            n -= n % P
            if n == 0:
                continue
            src = src_all[: n * es].view(dtype)
            dst = dst_all[: n * es].view(dtype)
            src.copy_(torch.randn(n, device=dev).to(dtype))
            ref = src.clone()
            iters = 20 if nbytes <= (16 << 20) else 5
            for op, nccl_op in (("sum", dist.ReduceOp.SUM), ("max", dist.ReduceOp.MAX)):
                rt.reduce(dst, src, op)
                dist.all_reduce(ref, op=nccl_op)
                torch.cuda.synchronize()
                # bf16: NCCL rounds to bf16 at every hop of its ring, this kernel accumulates in fp32 and rounds once
                good = torch.allclose(dst.float(), ref.float(), rtol=2e-2 if es == 2 else 1e-5, atol=0.3 if es == 2 else 1e-4)
                if not good:
                    print(f"[pe {me}] allreduce_{op} {dtype} {n * es} B: max diff {(dst.float() - ref.float()).abs().max().item()}", flush=True)
                    failed.append({"pe": me, "op": f"allreduce_{op}", "dtype": str(dtype), "bytes": n * es})
                ok_all &= bool(good)
                ref.copy_(src)
                us = timed(lambda: rt.reduce(dst, src, op), iters, rt)
                us_n = timed(lambda: dist.all_reduce(ref, op=nccl_op), iters, rt)
                ref.copy_(src)
                busbw = 2 * (P - 1) / P * n * es / us / 1e3
                rows.append({"op": f"allreduce_{op}", "dtype": str(dtype).split(".")[-1], "bytes": n * es, "us": us,
                             "nccl_us": us_n, "busbw_GBps": busbw, "nccl_busbw_GBps": 2 * (P - 1) / P * n * es / us_n / 1e3,
                             "ok": bool(good)})
            # reduce-scatter (sum)
            per = n // P
            rs_dst = dst[:per]
            rs_ref = torch.empty(per, device=dev, dtype=dtype)
            rt.reduce_scatter(rs_dst, src, "sum")
            dist.reduce_scatter_tensor(rs_ref, src)
            torch.cuda.synchronize()
            good = torch.allclose(rs_dst.float(), rs_ref.float(), rtol=2e-2 if es == 2 else 1e-5, atol=0.3 if es == 2 else 1e-4)
            if not good:
                print(f"[pe {me}] reduce_scatter {dtype} {n * es} B: max diff {(rs_dst.float() - rs_ref.float()).abs().max().item()}", flush=True)
                failed.append({"pe": me, "op": "reduce_scatter", "dtype": str(dtype), "bytes": n * es})
            ok_all &= bool(good)
            us = timed(lambda: rt.reduce_scatter(rs_dst, src, "sum"), iters, rt)
            us_n = timed(lambda: dist.reduce_scatter_tensor(rs_ref, src), iters, rt)
            rows.append({"op": "reduce_scatter_sum", "dtype": str(dtype).split(".")[-1], "bytes": n * es, "us": us, "nccl_us": us_n,
                         "busbw_GBps": (P - 1) / P * n * es / us / 1e3, "ok": bool(good)})
    # data movement: fcollect and alltoall (bytes = per-PE total buffer)
    for nbytes in sizes:
        blk = nbytes // P
        blk -= blk % 16
        if blk == 0:
            continue
        src = src_all[:blk]
        dst = dst_all[: blk * P]
        src.copy_(torch.randint(0, 256, (blk,), device=dev, dtype=torch.uint8))
        ref = torch.empty(blk * P, device=dev, dtype=torch.uint8)
        iters = 20 if nbytes <= (16 << 20) else 5
        rt.fcollect(dst, src)
        dist.all_gather_into_tensor(ref, src)
        torch.cuda.synchronize()
        good = torch.equal(dst, ref)
        if not good:
            bad = (dst != ref).nonzero()
            print(f"[pe {me}] fcollect {blk * P} B: {bad.shape[0]} bytes differ, first at {int(bad[0])} (block {int(bad[0]) // blk})", flush=True)
            failed.append({"pe": me, "op": "fcollect", "bytes": blk * P})
        ok_all &= bool(good)
        us = timed(lambda: rt.fcollect(dst, src), iters, rt)
        us_n = timed(lambda: dist.all_gather_into_tensor(ref, src), iters, rt)
        rows.append({"op": "fcollect", "bytes": blk * P, "us": us, "nccl_us": us_n, "busbw_GBps": (P - 1) * blk / us / 1e3,
                     "ok": bool(good)})
        a_src = src_all[: blk * P]
        a_src.copy_(torch.randint(0, 256, (blk * P,), device=dev, dtype=torch.uint8))
        rt.alltoall(dst, a_src)
        dist.all_to_all_single(ref, a_src)
        torch.cuda.synchronize()
        good = torch.equal(dst, ref)
        if not good:
            bad = (dst != ref).nonzero()
            print(f"[pe {me}] alltoall {blk * P} B: {bad.shape[0]} bytes differ, first at {int(bad[0])} (block {int(bad[0]) // blk})", flush=True)
            failed.append({"pe": me, "op": "alltoall", "bytes": blk * P})
        ok_all &= bool(good)
        us = timed(lambda: rt.alltoall(dst, a_src), iters, rt)
        us_n = timed(lambda: dist.all_to_all_single(ref, a_src), iters, rt)
        rows.append({"op": "alltoall", "bytes": blk * P, "us": us, "nccl_us": us_n, "busbw_GBps": (P - 1) * blk / us / 1e3,
                     "ok": bool(good)})
    # ---- launch-bound sizes replayed from a CUDA graph (the runtime follows the capturing stream) ----
    if args.graph:
        us = timed_graph(lambda: rt.barrier_all(), 50, rt)
        one = torch.zeros(1, device=dev)
        us_n = timed_graph(lambda: dist.all_reduce(one), 20, rt)   # dist.barrier() cannot be captured: a 4-byte all_reduce stands in
        rows.append({"op": "barrier_graph", "bytes": 0, "us": us, "nccl_us": us_n})
        for nbytes in (1024, 16384, 65536, 262144, 1 << 20):
            if nbytes > args.max_bytes:
                continue
            n = nbytes // 4
            n -= n % P
            src = src_all[: n * 4].view(torch.float32)
            dst = dst_all[: n * 4].view(torch.float32)
            src.copy_(torch.randn(n, device=dev))
            ref = src.clone()
            us = timed_graph(lambda: rt.reduce(dst, src, "sum"), 20, rt)
            us_n = timed_graph(lambda: dist.all_reduce(ref), 20, rt)
            rows.append({"op": "allreduce_sum_graph", "dtype": "float32", "bytes": n * 4, "us": us, "nccl_us": us_n})
    # ---- sub-teams: all teams of a size run their collective at the same time (team k = PEs [k*ts, (k+1)*ts)) ----
    for ts in [int(v) for v in args.team_sizes.split(",") if v]:
        if ts < 2 or ts >= P or P % ts:
            continue
        mine, group = None, None
        rt.synchronize()
        rt.set_blocking(True)                          # team creation is a host-synchronous collective
        for k in range(P // ts):                       # every PE takes part in every split, like every rank in every new_group
            t = rt.team_split_strided(None, k * ts, 1, ts)
            g = dist.new_group(list(range(k * ts, (k + 1) * ts)))
            if t.valid:
                mine, group = t, g
        rt.set_blocking(False)
        us = timed(lambda: mine.sync(), 50, rt)
        rows.append({"op": "team_sync", "team": ts, "bytes": 0, "us": us})
        for nbytes in [s_ for s_ in sizes if s_ in (1024, 65536, 1 << 20, 16 << 20, 256 << 20)]:
            n = nbytes // 4
            n -= n % ts
            src = src_all[: n * 4].view(torch.float32)
            dst = dst_all[: n * 4].view(torch.float32)
            src.copy_(torch.randn(n, device=dev))
            ref = src.clone()
            rt.reduce(dst, src, "sum", team=mine)
            dist.all_reduce(ref, group=group)
            torch.cuda.synchronize()
            good = torch.allclose(dst, ref, rtol=1e-5, atol=1e-4)
            ok_all &= bool(good)
            iters = 20 if nbytes <= (16 << 20) else 5
            us = timed(lambda: rt.reduce(dst, src, "sum", team=mine), iters, rt)
            us_n = timed(lambda: dist.all_reduce(ref, group=group), iters, rt)
            rows.append({"op": "allreduce_sum", "team": ts, "dtype": "float32", "bytes": n * 4, "us": us, "nccl_us": us_n,
                         "busbw_GBps": 2 * (ts - 1) / ts * n * 4 / us / 1e3, "nccl_busbw_GBps": 2 * (ts - 1) / ts * n * 4 / us_n / 1e3,
                         "ok": bool(good)})
            blk = (nbytes // ts) - (nbytes // ts) % 16
            if blk:
                fsrc, fdst = src_all[:blk], dst_all[: blk * ts]
                fref = torch.empty(blk * ts, device=dev, dtype=torch.uint8)
                rt.fcollect(fdst, fsrc, team=mine)
                dist.all_gather_into_tensor(fref, fsrc, group=group)
                torch.cuda.synchronize()
                good = torch.equal(fdst, fref)
                ok_all &= bool(good)
                us = timed(lambda: rt.fcollect(fdst, fsrc, team=mine), iters, rt)
                us_n = timed(lambda: dist.all_gather_into_tensor(fref, fsrc, group=group), iters, rt)
                rows.append({"op": "fcollect", "team": ts, "bytes": blk * ts, "us": us, "nccl_us": us_n,
                             "busbw_GBps": (ts - 1) * blk / us / 1e3, "ok": bool(good)})
        rt.synchronize()
        mine.destroy()
    rt.synchronize()
    rt.set_blocking(True)
    okt = torch.tensor([int(ok_all)], device=dev)
    dist.all_reduce(okt, op=dist.ReduceOp.MIN)
    all_failed = [f for fl in rt.bootstrap.allgather(failed, tag="coll-bench-failed") for f in fl] if P > 1 else failed
    if me == 0:
        out = {"n_pes": P, "all_ok": bool(okt.item()), "failed_checks": all_failed, "rows": rows}
        for r in rows:
            print(json.dumps(r))
        if args.out:
            os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
            with open(args.out, "w") as f:
                json.dump(out, f)
    shmem.finalize()
    dist.destroy_process_group()
    if not bool(okt.item()):
        raise SystemExit(1)


if __name__ == "__main__":
    main()
