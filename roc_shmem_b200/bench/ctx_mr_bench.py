"""Host multi-context message rate and bandwidth: T host threads, each with a context of its own, issue windows of
64 non-blocking puts followed by the context's quiet.

    python -m roc_shmem_b200.bench.ctx_mr_bench [--backend device|cpu] [--threads 1,2,4,8] [--out file.json]
    torchrun --nproc-per-node 2 -m roc_shmem_b200.bench.ctx_mr_bench          (PE 0 puts to PE 1)

Measurement definition: the reference's clients/sos_tests/put_ctx_mbw_mr.cpp:44-170 (OpenMP threads, one context
per thread, window 64, message rate in Mmsg/s and bandwidth in MB/s per message size).  On the NVLink backend a
context is a CUDA stream, so the threads' copies proceed independently; with one rank the target is the PE itself.
"""
from __future__ import annotations

import argparse
import json
import os
import threading
import time

import torch

import roc_shmem_b200 as shmem

WINDOW = 64


def run(rt, peer: int, n_threads: int, size: int, loops: int) -> tuple[float, float]:
    """Returns (Mmsg/s, MB/s) over all threads."""
    on_gpu = rt.device.type == "cuda"
    sym = rt.zeros((n_threads * WINDOW * size,), torch.uint8)
    srcs = [torch.ones(WINDOW * size, dtype=torch.uint8, device=rt.device) for _ in range(n_threads)]
    start, done = threading.Barrier(n_threads + 1), threading.Barrier(n_threads + 1)
    errs: list[BaseException] = []

    def work(t: int) -> None:
        try:
            if on_gpu:
                torch.cuda.set_device(rt.device)
            with rt.ctx_create(shmem.CTX_SERIALIZED) as c:
                base = t * WINDOW * size
                for phase in range(2):                      # 0 = warm-up, 1 = timed
                    if phase == 1:
                        start.wait()
                    for _ in range(loops if phase else 2):
                        for i in range(WINDOW):
                            c.put(sym[base + i * size: base + (i + 1) * size], srcs[t][i * size:(i + 1) * size], peer, nbi=True)
                        c.quiet()
                done.wait()
        except BaseException as e:  # noqa: BLE001
            errs.append(e)
            for b in (start, done):
                b.abort()
    ths = [threading.Thread(target=work, args=(t,)) for t in range(n_threads)]
    for th in ths:
        th.start()
    try:
        start.wait()
        t0 = time.perf_counter()
        done.wait()
        dt = time.perf_counter() - t0
    except threading.BrokenBarrierError:
        dt = float("nan")
    for th in ths:
        th.join()
    if errs:
        raise errs[0]
    rt.free(sym)
    msgs = n_threads * loops * WINDOW
    return msgs / dt / 1e6, msgs * size / dt / 1e6


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default="device" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--threads", default="1,2,4,8")
    ap.add_argument("--sizes", default="8,64,1024,16384,262144")
    ap.add_argument("--loops", type=int, default=20)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    kw = {"device": local} if args.backend != "cpu" else {}
    if args.backend != "cpu":
        torch.cuda.set_device(local)
    if world == 1:
        kw.update(rank=0, world_size=1)
    rt = shmem.init(args.backend, heap_bytes=512 << 20, **kw)
    me, n = rt.my_pe, rt.n_pes
    peer = 1 % n
    rows = []
    for size in [int(v) for v in args.sizes.split(",")]:
        for nt in [int(v) for v in args.threads.split(",")]:
            rt.barrier_all()
            if me == 0:
                mr, bw = run(rt, peer, nt, size, args.loops)
                rows.append({"threads": nt, "bytes": size, "Mmsg_s": round(mr, 4), "MB_s": round(bw, 2)})
                print(json.dumps(rows[-1]), flush=True)
            else:
                rt.free(rt.zeros((nt * WINDOW * size,), torch.uint8))     # the collective allocation and free of PE 0's run()
    rt.barrier_all()
    if me == 0 and args.out:
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        with open(args.out, "w") as f:
            json.dump({"backend": args.backend, "n_pes": n, "window": WINDOW, "rows": rows}, f)
    shmem.finalize()


if __name__ == "__main__":
    main()
