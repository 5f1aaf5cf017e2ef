"""Llama-style gated MLP block, tensor-parallel with sequence-parallel activations.

    x_shard [M/P, H] --all-gather→GEMM--> gu [M, 2F/P] --SwiGLU--> h [M, F/P]
            --GEMM→reduce-scatter--> y_shard [M/P, H]

Both collectives run inside the tcgen05 GEMM kernels (``ops.fused_tp``); the backward pass uses the
same two fused kernels with the transposed weights for the data gradients and the transposed-operand
(MN-major) GEMM for the weight gradients, so no activation is ever transposed in memory.  Default
dimensions are Llama-3-70B's (hidden 8192, FFN 28672).  The reference is a communication runtime and has
no model code; this block is the tensor-parallel workload its device API is meant to serve.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from ..ops.moe import grouped_gemm_tn, interleave_gate_up, moe_lib
from ..parallel.tp import ColumnParallelLinear, RowParallelLinear


class LlamaMLP:
    """Weights of this rank: ``w13`` [2F/P, H] (gate/up rows interleaved in groups of 32, see
    ``interleave_gate_up``) and ``w2`` [H, F/P]."""

    def __init__(self, rt, hidden: int = 8192, ffn: int = 28672, max_tokens: int = 8192, training: bool = True):
        P = rt.n_pes
        if ffn % P or (ffn // P) % 256 or hidden % 256 or max_tokens % (256 * P):
            raise ValueError("needs hidden % 256 == 0, (ffn / PEs) % 256 == 0 and tokens % (256 * PEs) == 0")
        self.rt, self.P, self.H, self.F, self.Fp, self.M = rt, P, hidden, ffn, ffn // P, max_tokens
        self.training = training
        dev, bf = rt.device, torch.bfloat16
        M, H, Fp = self.M, hidden, self.Fp
        self.up = ColumnParallelLinear(rt, H, 2 * Fp, M)            # gathers x, produces gu
        self.down = RowParallelLinear(rt, Fp, H, M)                 # consumes h, scatters y
        self.w13, self.w2 = self.up.weight, self.down.weight
        self.gu = self.up.out
        self.h = torch.empty((M, Fp), dtype=bf, device=dev)
        self.rows = torch.full((1,), M, dtype=torch.int32, device=dev)
        self.lib = moe_lib()
        self.launches = 0
        if training:
            self.w13_t = torch.empty((H, 2 * Fp), dtype=bf, device=dev)
            self.w2_t = torch.empty((Fp, H), dtype=bf, device=dev)
            self.dgrad_h = ColumnParallelLinear(rt, H, Fp, M)       # gathers dy, produces dh = dy @ W2
            self.dgrad_x = RowParallelLinear(rt, 2 * Fp, H, M)      # dx = reduce_scatter(dgu @ W13)
            self.dgu = torch.empty((M, 2 * Fp), dtype=bf, device=dev)
            self.dw13 = torch.empty((2 * Fp, H), dtype=bf, device=dev)
            self.dw2 = torch.empty((H, Fp), dtype=bf, device=dev)

    # ---- weights -------------------------------------------------------------------------
    def load(self, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> None:
        """This rank's shards: gate/up [F/P, H], down [H, F/P]."""
        self.w13.copy_(interleave_gate_up(w_gate.to(torch.bfloat16), w_up.to(torch.bfloat16)))
        self.w2.copy_(w_down)
        self.sync_transposes()

    def sync_transposes(self) -> None:
        """Refresh the transposed weight copies the data-gradient GEMMs read (call after a weight update)."""
        if self.training:
            self.w13_t.copy_(self.w13.t())
            self.w2_t.copy_(self.w2.t())

    def _chk(self, st: int, what: str) -> None:
        if st != 0:
            raise RuntimeError(f"{what} failed ({st}): {self.lib.bshmem_moe_last_error().decode()}")

    # ---- forward / backward ------------------------------------------------------------------
    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        s = torch.cuda.current_stream().cuda_stream
        self.up(x_shard)
        self._chk(self.lib.bshmem_moe_swiglu_fwd(self.gu.data_ptr(), self.rows.data_ptr(), 1, self.M, self.Fp, self.h.data_ptr(), s),
                  "swiglu")
        y = self.down(self.h)
        self.launches += 3
        return y

    __call__ = forward

    def backward(self, dy_shard: torch.Tensor) -> torch.Tensor:
        """Returns dx_shard [M/P, H]; weight gradients land in ``dw13`` / ``dw2``.  Must follow forward()."""
        assert self.training
        s = torch.cuda.current_stream().cuda_stream
        dh = self.dgrad_h(dy_shard, weight=self.w2_t)                              # [M, F/P], gathers dy
        grouped_gemm_tn(self.dgrad_h.gathered, self.h, self.dw2, 1, self.rows)     # dW2 = dy^T h
        self._chk(self.lib.bshmem_moe_swiglu_bwd(self.gu.data_ptr(), dh.data_ptr(), self.rows.data_ptr(), 1, self.M, self.Fp,
                                                 self.dgu.data_ptr(), s), "swiglu bwd")
        grouped_gemm_tn(self.dgu, self.up.gathered, self.dw13, 1, self.rows)       # dW13 = dgu^T x
        dx = self.dgrad_x(self.dgu, weight=self.w13_t)
        self.launches += 5
        return dx

    def check(self) -> None:
        for layer in (self.up, self.down) + ((self.dgrad_h, self.dgrad_x) if self.training else ()):
            layer.check()
        site = self.lib.bshmem_moe_gemm_error_site(1)
        if site:
            raise RuntimeError(f"a bounded in-kernel wait ran out (site {site})")


class _LlamaMLPFn(torch.autograd.Function):
    """autograd bridge: the block's hand-written backward supplies every gradient."""

    @staticmethod
    def forward(ctx, x, w13, w2, block):
        ctx.block = block
        return block.forward(x).clone()

    @staticmethod
    def backward(ctx, dy):
        block = ctx.block
        dx = block.backward(dy.contiguous())
        return dx.clone(), block.dw13.clone(), block.dw2.clone(), None


class LlamaMLPModule(torch.nn.Module):
    """``torch.nn.Module`` face of ``LlamaMLP``: parameters alias the block's weight buffers, gradients come
    from the block's own backward kernels.  Call ``block.sync_transposes()`` (or ``after_step()``) after
    every optimiser step."""

    def __init__(self, rt, hidden: int = 8192, ffn: int = 28672, max_tokens: int = 8192):
        super().__init__()
        self.block = LlamaMLP(rt, hidden, ffn, max_tokens, training=True)
        self.w13 = torch.nn.Parameter(self.block.w13)
        self.w2 = torch.nn.Parameter(self.block.w2)

    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        return _LlamaMLPFn.apply(x_shard, self.w13, self.w2, self.block)

    def after_step(self) -> None:
        self.block.sync_transposes()


def reference_mlp(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """Plain fp32 PyTorch math of the whole (unsharded) block, for tests."""
    return (torch.nn.functional.silu(x @ w_gate.t()) * (x @ w_up.t())) @ w_down.t()
