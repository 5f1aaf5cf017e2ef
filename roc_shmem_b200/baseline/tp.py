"""Baseline for the fused tensor-parallel ops: cuBLAS (torch.matmul) + NCCL collectives
on the same buffers.  A path that only calls NCCL is the baseline, not the product.

Two forms of each op: back to back on one stream (what `torch` code does by default),
and chunked over two streams so that the collective of chunk i overlaps the GEMM of
chunk i+1 (what a user would write before reaching for a fused kernel).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _world() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def gemm_reduce_scatter(x: torch.Tensor, w: torch.Tensor, partial: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """partial[M, N] = x @ w.T ; out[M/P, N] = reduce_scatter(partial) over the default group.
    With one rank the collective is the identity and the GEMM writes `out` directly."""
    if _world() == 1:
        torch.matmul(x, w.t(), out=out)
        return out
    torch.matmul(x, w.t(), out=partial)
    dist.reduce_scatter_tensor(out, partial)
    return out


def all_gather_gemm(x_shard: torch.Tensor, w: torch.Tensor, gathered: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """gathered[M, K] = all_gather(x_shard) ; out[M, N] = gathered @ w.T"""
    if _world() == 1:
        torch.matmul(x_shard, w.t(), out=out)
        return out
    dist.all_gather_into_tensor(gathered, x_shard)
    torch.matmul(gathered, w.t(), out=out)
    return out


class OverlappedGemmReduceScatter:
    """GEMM → reduce-scatter in `chunks` row chunks: chunk i's NCCL reduce-scatter runs on a side stream
    while cuBLAS computes chunk i+1.  Rank r ends up with rows r*M/(C*P) .. of every chunk (a row
    permutation of the unchunked result: `rows()` gives the global row index of each output row)."""

    def __init__(self, M: int, N: int, device, chunks: int = 4):
        self.P = _world()
        self.C = chunks if M % (chunks * self.P) == 0 else 1
        self.M, self.N = M, N
        self.partial = torch.empty(M, N, device=device, dtype=torch.bfloat16)
        self.out = torch.empty(M // self.P, N, device=device, dtype=torch.bfloat16)
        self.side = torch.cuda.Stream(device=device)
        self.ev = [torch.cuda.Event() for _ in range(self.C)]
        self.done = torch.cuda.Event()

    def rows(self, rank: int) -> torch.Tensor:
        mc = self.M // self.C
        per = mc // self.P
        return torch.cat([torch.arange(c * mc + rank * per, c * mc + (rank + 1) * per) for c in range(self.C)])

    def __call__(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        main = torch.cuda.current_stream()
        if self.P == 1:
            torch.matmul(x, w.t(), out=self.out)
            return self.out
        mc = self.M // self.C
        per = mc // self.P
        self.side.wait_stream(main)          # earlier readers of `out` / writers of x are ordered before the side stream
        for c in range(self.C):
            torch.matmul(x[c * mc:(c + 1) * mc], w.t(), out=self.partial[c * mc:(c + 1) * mc])
            self.ev[c].record(main)
            with torch.cuda.stream(self.side):
                self.side.wait_event(self.ev[c])
                dist.reduce_scatter_tensor(self.out[c * per:(c + 1) * per], self.partial[c * mc:(c + 1) * mc])
        self.done.record(self.side)
        main.wait_event(self.done)
        return self.out


class OverlappedAllGatherGemm:
    """all-gather → GEMM in `chunks` row chunks of every rank's shard: the NCCL all-gather of chunk i+1 runs on a
    side stream while cuBLAS multiplies chunk i.  Output rows come out chunk-major (`rows()` maps them back)."""

    def __init__(self, M: int, N: int, K: int, device, chunks: int = 4):
        self.P = _world()
        self.C = chunks if (M // self.P) % chunks == 0 else 1
        self.M, self.N, self.K = M, N, K
        self.gathered = torch.empty(M, K, device=device, dtype=torch.bfloat16)
        self.out = torch.empty(M, N, device=device, dtype=torch.bfloat16)
        self.side = torch.cuda.Stream(device=device)
        self.ev = [torch.cuda.Event() for _ in range(self.C)]

    def rows(self) -> torch.Tensor:
        per = self.M // self.P // self.C
        idx = []
        for c in range(self.C):
            for r in range(self.P):
                base = r * (self.M // self.P) + c * per
                idx.append(torch.arange(base, base + per))
        return torch.cat(idx)

    def __call__(self, x_shard: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        main = torch.cuda.current_stream()
        if self.P == 1:
            torch.matmul(x_shard, w.t(), out=self.out)
            return self.out
        per = x_shard.shape[0] // self.C
        blk = per * self.P
        self.side.wait_stream(main)
        with torch.cuda.stream(self.side):
            for c in range(self.C):
                dist.all_gather_into_tensor(self.gathered[c * blk:(c + 1) * blk], x_shard[c * per:(c + 1) * per])
                self.ev[c].record(self.side)
        for c in range(self.C):
            main.wait_event(self.ev[c])
            torch.matmul(self.gathered[c * blk:(c + 1) * blk], w.t(), out=self.out[c * blk:(c + 1) * blk])
        return self.out
