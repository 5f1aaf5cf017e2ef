"""Device collectives of a local group (all PEs of the job on ONE GPU, one cooperative launch per collective):
timing and a correctness check of allreduce / reduce-scatter / fcollect / alltoall without any NVLink hop.

    python -m roc_shmem_b200.bench.coll_local_bench [--pes 4] [--bytes 67108864] [--op allreduce] [--dtype float32] [--iters 5]

Used for single-GPU profiler captures of the collective kernels (HBM bytes against algorithmic bytes); the
multi-GPU numbers come from coll_bench.  The reference's collectives cannot run on one device at all.
"""
from __future__ import annotations

import argparse
import json

import torch

from roc_shmem_b200 import gpu
from roc_shmem_b200.utils import dtypes as D


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--pes", type=int, default=4)
    ap.add_argument("--bytes", type=int, default=64 << 20, help="per-PE vector (allreduce) / total per PE (others)")
    ap.add_argument("--op", default="allreduce", choices=["allreduce", "reduce_scatter", "fcollect", "alltoall"])
    ap.add_argument("--dtype", default="float32", choices=["float32", "bfloat16"])
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--ctas", type=int, default=32)
    args = ap.parse_args()
    dt = getattr(torch, args.dtype)
    es = 2 if dt == torch.bfloat16 else 4
    P = args.pes
    n = args.bytes // es
    n -= n % (P * 8)
    group = gpu.LocalGroup(P, heap_bytes=4 * args.bytes + (256 << 20))
    try:
        src = group.empty((n,), dt)
        dst = group.empty((n,), dt)
        for i, s_ in enumerate(src):
            s_.copy_(torch.randn(n, device="cuda").to(dt))
        kind, count = {"allreduce": (gpu.COLL_REDUCE, n), "reduce_scatter": (gpu.COLL_REDUCE_SCATTER, n // P),
                       "fcollect": (gpu.COLL_FCOLLECT, n // P * es), "alltoall": (gpu.COLL_ALLTOALL, n // P * es)}[args.op]

        def call():
            group.collective(kind, dst, src, count, dtype=dt, op=D.SUM, ctas=args.ctas)
        call()
        torch.cuda.synchronize()
        ok = True
        if args.op == "allreduce":
            ref = torch.stack([s_.float() for s_ in src]).sum(0)
            ok = all(torch.allclose(d.float(), ref, rtol=2e-2 if es == 2 else 1e-5, atol=1e-2 if es == 2 else 1e-4) for d in dst)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            call()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / args.iters
        print(json.dumps({"op": args.op, "pes": P, "dtype": args.dtype, "bytes_per_pe": n * es, "us": round(us, 2), "ok": bool(ok),
                          "note": "includes the per-call table allocation of the group entry; all PEs share one GPU's HBM"}))
    finally:
        group.close()


if __name__ == "__main__":
    main()
