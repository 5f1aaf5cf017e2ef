"""Tensor-parallel linear layers whose collective is fused into the GEMM kernel.

``RowParallelLinear``  : y = reduce_scatter_M( x_shard @ W_shard.T )   (MLP down-projection)
``ColumnParallelLinear``: y_shard = all_gather_M(x_shard) @ W_shard.T   (MLP gate/up projection)

Both run hand-written sm_100a kernels (tcgen05 + TMEM + TMA) that move the tiles
over NVLink peer memory from inside the GEMM; with one PE they reduce to the plain
GEMM.  The reference has no such layer (it is a communication library only); these
are the north-star workloads built on its device API shape.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops.gemm import gemm_bf16, gemm_error_site


class RowParallelLinear:
    """x: [M, K/P] (this rank's K shard) ; weight: [N, K/P] ; returns this rank's [M/P, N] rows of
    sum over ranks of x_r @ w_r.T."""

    def __init__(self, rt, in_features_per_rank: int, out_features: int, max_tokens: int,
                 dtype: torch.dtype = torch.bfloat16):
        if dtype != torch.bfloat16:
            raise ValueError("bf16 only (see ops.gemm_fp8 for the block-scaled fp8 variant)")
        self.rt = rt
        self.P = rt.n_pes
        self.K, self.N, self.M = in_features_per_rank, out_features, max_tokens
        if self.M % self.P:
            raise ValueError("token count must divide by the number of PEs")
        dev = rt.device
        self.weight = torch.empty((self.N, self.K), dtype=dtype, device=dev)
        self.x_bufs = None          # step_from_host() allocates its double-buffered inputs on first use
        self._step = 0
        self._launches = 0
        if self.P == 1:
            self.out = torch.empty((self.M, self.N), dtype=dtype, device=dev)
            self.algorithm = ("tcgen05 GEMM on CTA pairs (cta_group::2, 256x256x64 tiles, 6-stage TMA ring, two TMEM "
                              "accumulator stages); 1 PE: no collective")
            self._fused = None
        else:
            from ..ops.fused_tp import GemmReduceScatter
            self._fused = GemmReduceScatter(rt, self.M, self.N, self.K)
            self.out = self._fused.out
            self.algorithm = self._fused.algorithm

    def forward(self, x: torch.Tensor, weight: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        w = self.weight if weight is None else weight
        out = self.out if out is None else out
        if self._fused is None:
            gemm_bf16(x, w, out)
            self._launches += 1
            return out
        self._launches += self._fused(x, w, out)
        return out

    __call__ = forward

    def step_from_host(self, x_host: torch.Tensor, result_host: torch.Tensor) -> None:
        """One serving-style step: pinned host activations -> device (copy stream, double-buffered so that
        the copy of the next step overlaps this step's kernel), the layer, then the first row of the result
        back into the pinned `result_host` ([N] bf16)."""
        if self.x_bufs is None:
            # double-buffered device inputs + a copy stream: the host->device copy of step i+1 overlaps step i
            dev = self.rt.device
            self.x_bufs = [torch.empty((self.M, self.K), dtype=torch.bfloat16, device=dev) for _ in range(2)]
            self.copy_stream = torch.cuda.Stream(device=dev)
            self.copied = [torch.cuda.Event() for _ in range(2)]
            self.consumed = [torch.cuda.Event() for _ in range(2)]
        i = self._step & 1
        main = torch.cuda.current_stream()
        with torch.cuda.stream(self.copy_stream):
            if self._step >= 2:
                self.copy_stream.wait_event(self.consumed[i])     # the kernel that read this buffer is done
            self.x_bufs[i].copy_(x_host, non_blocking=True)
            self.copied[i].record(self.copy_stream)
        main.wait_event(self.copied[i])
        y = self.forward(self.x_bufs[i])
        self.consumed[i].record(main)
        result_host.copy_(y[0], non_blocking=True)
        self._step += 1

    def reset_launch_count(self) -> None:
        self._launches = 0

    def launch_count(self) -> int:
        return self._launches

    def check(self) -> None:
        site = gemm_error_site()
        if site:
            raise RuntimeError(f"a bounded in-kernel wait ran out (site {site})")
        if self._fused is not None:
            self._fused.check()


class ColumnParallelLinear:
    """x_shard: [M/P, K] (this rank's token rows) ; weight: [N/P, K] ; returns [M, N/P] =
    all_gather_rows(x) @ w.T.  The caller writes its rows into ``self.x_shard`` (a view of the symmetric
    gathered buffer) or passes them to forward(), which copies them there; after the call ``self.gathered``
    holds all M rows (reused by the weight-gradient GEMM of a backward pass)."""

    def __init__(self, rt, in_features: int, out_features_per_rank: int, max_tokens: int):
        self.rt, self.P = rt, rt.n_pes
        self.K, self.N, self.M = in_features, out_features_per_rank, max_tokens
        if self.M % self.P:
            raise ValueError("token count must divide by the number of PEs")
        dev = rt.device
        self.weight = torch.empty((self.N, self.K), dtype=torch.bfloat16, device=dev)
        self._launches = 0
        if self.P == 1:
            self.gathered = torch.empty((self.M, self.K), dtype=torch.bfloat16, device=dev)
            self.x_shard = self.gathered
            self.out = torch.empty((self.M, self.N), dtype=torch.bfloat16, device=dev)
            self._fused = None
            self.algorithm = "tcgen05 GEMM; 1 PE: no collective"
        else:
            from ..ops.fused_tp import AllGatherGemm
            self._fused = AllGatherGemm(rt, self.M, self.N, self.K)
            self.gathered, self.x_shard, self.out = self._fused.xg, self._fused.x_shard, self._fused.out
            self.algorithm = self._fused.algorithm

    def forward(self, x_shard: Optional[torch.Tensor] = None, weight: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        w = self.weight if weight is None else weight
        out = self.out if out is None else out
        if x_shard is not None and x_shard.data_ptr() != self.x_shard.data_ptr():
            self.x_shard.copy_(x_shard)
        if self._fused is None:
            gemm_bf16(self.gathered, w, out)
            self._launches += 1
        else:
            self._launches += self._fused(w, out)
        return out

    __call__ = forward

    def launch_count(self) -> int:
        return self._launches

    def check(self) -> None:
        site = gemm_error_site()
        if site:
            raise RuntimeError(f"a bounded in-kernel wait ran out (site {site})")
        if self._fused is not None:
            self._fused.check()


def smoke_step(rt) -> None:
    """Tiny forward of the flagship layer (used by the driver's smoke test)."""
    layer = RowParallelLinear(rt, in_features_per_rank=256, out_features=512, max_tokens=512)
    layer.weight.copy_((torch.randn(512, 256, device=rt.device) * 0.05).to(torch.bfloat16))
    x = torch.randn(512, 256, device=rt.device).to(torch.bfloat16)
    y = layer(x)
    torch.cuda.synchronize()
    layer.check()
    ref = x.float() @ layer.weight.float().t()
    assert (y.float() - ref).abs().max().item() < 0.05 * ref.abs().max().item() + 0.05
