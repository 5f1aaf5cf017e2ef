"""Byte-exact checks of the device collectives at 1 KiB .. MAX bytes (run under torchrun, one rank per GPU).

Every op runs in stream mode (calls only enqueue, like NCCL) several times back to back on buffers whose
contents are a closed form of (source PE, position), so a wrong or stale byte names its origin:
fcollect, alltoall, broadcast, int32 sum reduce-scatter and allreduce (exact in integer arithmetic).
Prints "COLL_EXACT_OK <rank>" on success; every failed check prints rank, op, size and the first bad position.
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import roc_shmem_b200 as shmem  # noqa: E402


def pattern(pe: int, n: int, dev, salt: int) -> torch.Tensor:
    """int32 values: a function of the source PE, the position and the repetition."""
    i = torch.arange(n, device=dev, dtype=torch.int64)
    return ((i * 2654435761 + pe * 40503 + salt * 97) % 1000003).to(torch.int32)


def first_bad(a: torch.Tensor, b: torch.Tensor) -> str:
    ne = (a != b).nonzero()
    if ne.numel() == 0:
        return "none"
    k = int(ne[0])
    return f"{ne.shape[0]} bad of {a.numel()}, first at {k}: got {int(a[k])} want {int(b[k])}"


def main() -> None:
    local = int(os.environ.get("LOCAL_RANK", 0))
    max_bytes = int(os.environ.get("COLL_EXACT_MAX_BYTES", str(64 << 20)))
    torch.cuda.set_device(local)
    rt = shmem.init("device", device=local, heap_bytes=int(max_bytes * 2.5) + (256 << 20), timeout_ms=10000,
                    coll_ctas=int(os.environ.get("COLL_EXACT_CTAS", "128")))
    me, P, dev = rt.my_pe, rt.n_pes, rt.device
    src_all = rt.empty((max_bytes // 4,), torch.int32, align=1024)
    dst_all = rt.empty((max_bytes // 4,), torch.int32, align=1024)
    rt.set_blocking(False)
    failures = []
    sizes, s = [], 1024
    while s <= max_bytes:
        sizes.append(s)
        s *= 4
    if sizes[-1] != max_bytes:
        sizes.append(max_bytes)
    salt = 0
    for nbytes in sizes:
        blk = nbytes // 4 // P            # int32 elements per block
        blk -= blk % 4                    # 16-byte granular blocks
        if blk == 0:
            continue
        for rep in range(3):              # back to back: a stale byte of the previous repetition shows up
            salt += 1
            # ---- fcollect ----
            src = src_all[:blk]
            dst = dst_all[: blk * P]
            src.copy_(pattern(me, blk, dev, salt))
            rt.fcollect(dst, src)
            want = torch.cat([pattern(k, blk, dev, salt) for k in range(P)])
            if not torch.equal(dst, want):
                failures.append(f"[pe {me}] fcollect {nbytes} B rep {rep}: {first_bad(dst, want)}")
            # ---- alltoall: block j of PE i holds pattern(i * P + j) ----
            a_src = src_all[: blk * P]
            for j in range(P):
                a_src[j * blk:(j + 1) * blk] = pattern(me * P + j, blk, dev, salt)
            rt.alltoall(dst, a_src)
            want = torch.cat([pattern(k * P + me, blk, dev, salt) for k in range(P)])
            if not torch.equal(dst, want):
                failures.append(f"[pe {me}] alltoall {nbytes} B rep {rep}: {first_bad(dst, want)}")
            # ---- reduce-scatter and allreduce, int32 sum (exact) ----
            n = blk * P
            r_src = src_all[:n]
            r_src.copy_(pattern(me, n, dev, salt))
            total = torch.zeros(n, device=dev, dtype=torch.int64)
            for k in range(P):
                total += pattern(k, n, dev, salt)
            total = total.to(torch.int32)
            rs_dst = dst_all[:blk]
            rt.reduce_scatter(rs_dst, r_src, "sum")
            if not torch.equal(rs_dst, total[me * blk:(me + 1) * blk]):
                failures.append(f"[pe {me}] reduce_scatter {nbytes} B rep {rep}: {first_bad(rs_dst, total[me * blk:(me + 1) * blk])}")
            ar_dst = dst_all[:n]
            rt.reduce(ar_dst, r_src, "sum")
            if not torch.equal(ar_dst, total):
                failures.append(f"[pe {me}] allreduce {nbytes} B rep {rep}: {first_bad(ar_dst, total)}")
            # ---- broadcast from the last PE (the root's dest stays untouched) ----
            b_src = src_all[:n]
            b_src.copy_(pattern(me + 100, n, dev, salt))
            b_dst = dst_all[:n]
            b_dst.fill_(-7)
            rt.broadcast(b_dst, b_src, P - 1)
            want = pattern(P - 1 + 100, n, dev, salt) if me != P - 1 else torch.full((n,), -7, device=dev, dtype=torch.int32)
            if not torch.equal(b_dst, want):
                failures.append(f"[pe {me}] broadcast {nbytes} B rep {rep}: {first_bad(b_dst, want)}")
    rt.synchronize()
    rt.set_blocking(True)
    for f in failures:
        print(f, flush=True)
    all_fail = rt.bootstrap.allgather(len(failures), tag="coll-exact") if P > 1 else [len(failures)]
    shmem.finalize()
    if sum(all_fail):
        raise SystemExit(1)
    print(f"COLL_EXACT_OK {me}", flush=True)


if __name__ == "__main__":
    main()
