"""Baseline for the fused tensor-parallel ops: cuBLAS (torch.matmul) + NCCL collectives
on the same buffers.  A path that only calls NCCL is the baseline, not the product."""
from __future__ import annotations

import torch
import torch.distributed as dist


def gemm_reduce_scatter(x: torch.Tensor, w: torch.Tensor, partial: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """partial[M, N] = x @ w.T ; out[M/P, N] = reduce_scatter(partial) over the default group."""
    torch.matmul(x, w.t(), out=partial)
    if dist.get_world_size() == 1:
        out.copy_(partial)
    else:
        dist.reduce_scatter_tensor(out, partial)
    return out


def all_gather_gemm(x_shard: torch.Tensor, w: torch.Tensor, gathered: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """gathered[M, K] = all_gather(x_shard) ; out[M, N] = gathered @ w.T"""
    if dist.get_world_size() == 1:
        gathered.copy_(x_shard)
    else:
        dist.all_gather_into_tensor(gathered, x_shard)
    torch.matmul(gathered, w.t(), out=out)
    return out
