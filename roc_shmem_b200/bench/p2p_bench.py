"""Device-initiated point-to-point sweep between PE pairs (latency and GB/s vs size).

    torchrun --nproc-per-node P -m roc_shmem_b200.bench.p2p_bench [--max-bytes 268435456] [--out file.json]

PE 0 is the initiator and PE `--peer` (default 1) the target (other PEs idle at the
barriers), as in the reference's functional tests
(clients/functional_tests/tester.cpp:566-586: only PE 0 launches).  Measured: putmem /
getmem at thread, warp and block scope and with bulk async copies over 1..132 issuing
CTAs, sizes 8 B .. 256 MiB of uniform random bytes (seed 0); one-way putmem_signal
bandwidth over the same CTA counts; 8-byte atomic_fetch_add rate over 1..132 CTAs;
p + wait_until ping-pong; putmem_signal ping-pong; 8-byte atomic latency; put_nbi
message rate.  Bandwidth is device time from CUDA events around the kernel.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

import roc_shmem_b200 as shmem
from roc_shmem_b200.utils import dtypes as D


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-bytes", type=int, default=256 << 20)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--out", default="")
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--peer", type=int, default=1, help="target PE of the sweep (PE 0 initiates)")
    ap.add_argument("--one", default="", help="SCOPE:CTAS:BYTES — run only that put a few times (profiler captures, one rank: the target is the PE itself)")
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    rt = shmem.init("device", device=local, heap_bytes=max(2 * args.max_bytes, 64 << 20) + (64 << 20))
    me, n = rt.my_pe, rt.n_pes
    dev = rt.device
    res = {"n_pes": n, "bandwidth": [], "latency": {}}
    tgt = args.peer if 0 < args.peer < n else (1 if n > 1 else 0)
    if n < 2:
        peer = 0
    else:
        peer = tgt if me == 0 else 0
    pair = (0, tgt)
    g = torch.Generator(device="cpu").manual_seed(0)
    sym = rt.empty((args.max_bytes,), torch.uint8)
    src = torch.randint(0, 256, (args.max_bytes,), dtype=torch.uint8, generator=g).to(dev)
    flag = rt.zeros((1,), torch.int64)
    sigs = rt.zeros((8,), torch.int64)
    target = rt.zeros((1,), torch.int64)
    amo_words = rt.zeros((65536,), torch.int64)
    rt.barrier_all()
    if args.one:
        scope, ctas, size = args.one.split(":")
        for _ in range(3):
            rt.rma_kernel(sym, src, peer, put=True, scope=scope, ctas=int(ctas), threads=128 if scope == "bulk" else 512, nbytes=int(size))
        rt.quiet()
        torch.cuda.synchronize()
        print(json.dumps({"one": args.one, "ok": bool(torch.equal(sym[: int(size)], src[: int(size)])) if n == 1 else None}))
        shmem.finalize()
        return

    # ---- latency micro-benchmarks (both PEs of the pair participate) ----
    if me in pair and n >= 2:
        iters = 200
        res["latency"]["pingpong_p_wait_us"] = rt.bench_pingpong(flag, peer, iters, me == 0)
    rt.barrier_all()
    if me in pair and n >= 2:
        for k, nb in enumerate((8, 1024, 65536)):
            # one fresh (zero) signal word per run: the values 1..iters must not meet a stale word
            res["latency"][f"put_signal_{nb}B_us"] = rt.bench_put_signal(sym, sigs[k:k + 1], nb, peer, 100, me == 0)
    rt.barrier_all()
    if me == 0:
        for name, op in (("fetch_add", D.AMO_FETCH_ADD), ("compare_swap", D.AMO_FETCH_CSWAP), ("swap", D.AMO_SWAP),
                         ("fetch", D.AMO_FETCH), ("add", D.AMO_ADD)):
            res["latency"][f"amo_{name}_us"] = rt.bench_amo(target, peer, 500, op)
        for size in (8, 64, 512):
            res["latency"][f"put_nbi_msgrate_{size}B_Mmsg_s"] = rt.bench_msgrate(sym, src, size, peer, 4, 8, 256)
    rt.barrier_all()

    # ---- bandwidth sweep: PE 0 drives ----
    sizes = []
    s = 8
    while s <= args.max_bytes:
        sizes.append(s)
        s *= 4 if args.quick else 2
    configs = [("block", 1, 512), ("block", 8, 512), ("block", 32, 512), ("block", 132, 512), ("warp", 32, 512),
               ("thread", 32, 256), ("bulk", 8, 128), ("bulk", 32, 128), ("bulk", 64, 128), ("bulk", 132, 128)]
    if args.quick:
        configs = [("block", 1, 512), ("block", 32, 512), ("block", 132, 512), ("warp", 32, 512), ("bulk", 32, 128),
                   ("bulk", 132, 128)]
    if me == 0:
        for op in ("put", "get"):
            for scope, ctas, threads in configs:
                for size in sizes:
                    if scope == "thread" and size > (64 << 20):
                        continue
                    if scope == "bulk" and size < (64 << 10):
                        continue
                    iters = args.iters if size <= (16 << 20) else max(3, args.iters // 3)
                    for _ in range(2):
                        rt.rma_kernel(sym, src, peer, put=(op == "put"), scope=scope, ctas=ctas, threads=threads, nbytes=size)
                    torch.cuda.synchronize()
                    rt.quiet()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for _ in range(iters):
                        rt.rma_kernel(sym, src, peer, put=(op == "put"), scope=scope, ctas=ctas, threads=threads, nbytes=size)
                    e1.record()
                    torch.cuda.synchronize()
                    us = e0.elapsed_time(e1) * 1e3 / iters
                    res["bandwidth"].append({"op": op, "scope": scope, "ctas": ctas, "threads": threads, "bytes": size,
                                             "us": round(us, 3), "GBps": round(size / us / 1e3, 2)})
        # host-initiated put / get (the copy engine moves the bytes): the peer-copy rate the device paths are held against
        rt.set_blocking(False)
        for op in ("host_put", "host_get"):
            for size in [x for x in sizes if x >= (64 << 10)]:
                iters = args.iters if size <= (16 << 20) else max(3, args.iters // 3)

                def one():
                    if op == "host_put":
                        rt.put(sym[:size], src[:size], peer, nbi=True)
                    else:
                        rt.get(src[:size], sym[:size], peer, nbi=True)
                one()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(iters):
                    one()
                e1.record()
                torch.cuda.synchronize()
                us = e0.elapsed_time(e1) * 1e3 / iters
                res["bandwidth"].append({"op": op, "scope": "copy_engine", "ctas": 0, "threads": 0, "bytes": size,
                                         "us": round(us, 3), "GBps": round(size / us / 1e3, 2)})
        rt.synchronize()
        rt.set_blocking(True)
        src.copy_(torch.randint(0, 256, (args.max_bytes,), dtype=torch.uint8,
                                generator=torch.Generator(device="cpu").manual_seed(0)).to(dev))   # host_get overwrote it
        # one-way putmem_signal bandwidth and 8-byte fetch-add rate as sweeps over the issuing CTAs
        res["put_signal_bandwidth"], res["amo_fetch_add_rate"] = [], []
        sig = sigs[7:8]
        for ctas in (1, 8, 32, 132):
            for size in [x for x in sizes if x >= 4096]:
                iters = 8 if size <= (16 << 20) else 3
                rt.put_signal_stream(sym, src, sig, size, peer, 2, ctas)
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                rt.put_signal_stream(sym, src, sig, size, peer, iters, ctas)
                e1.record()
                torch.cuda.synchronize()
                us = e0.elapsed_time(e1) * 1e3 / iters
                res["put_signal_bandwidth"].append({"ctas": ctas, "bytes": size, "us": round(us, 3), "GBps": round(size / us / 1e3, 2)})
        for ctas in (1, 2, 4, 8, 16, 32, 64, 132):
            for threads in (32, 256):
                mops = rt.bench_amo_rate(amo_words, peer, 64, ctas, threads)
                res["amo_fetch_add_rate"].append({"ctas": ctas, "threads": threads, "Mops": round(mops, 2)})
    rt.barrier_all()
    # verification of the last put (whole buffer) on the target
    if n >= 2:
        if me == 0:
            rt.rma_kernel(sym, src, peer, put=True, scope="block", ctas=64, threads=512, nbytes=args.max_bytes)
            rt.quiet()
        rt.barrier_all()
        if me == tgt:
            res_ok = bool(torch.equal(sym, torch.randint(0, 256, (args.max_bytes,), dtype=torch.uint8,
                                                         generator=torch.Generator(device="cpu").manual_seed(0)).to(dev)))
            ok_list = rt.bootstrap.allgather(res_ok, tag="p2p-ok")
        else:
            ok_list = rt.bootstrap.allgather(True, tag="p2p-ok")
        res["verified"] = all(ok_list)
    if me == 0:
        best = {}
        for r in res["bandwidth"]:
            k = r["op"]
            if r["bytes"] >= (64 << 20):
                best[k] = max(best.get(k, 0.0), r["GBps"])
                if r["scope"] == "bulk":
                    best[k + "_bulk"] = max(best.get(k + "_bulk", 0.0), r["GBps"])
        res["peak_GBps"] = best
        line = json.dumps(res)
        print(json.dumps({k: v for k, v in res.items() if k != "bandwidth"}), flush=True)
        if args.out:
            os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
            with open(args.out, "w") as f:
                f.write(line + "\n")
    shmem.finalize()


if __name__ == "__main__":
    main()
