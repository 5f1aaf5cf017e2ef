"""Mixtral-style sparse MoE block with expert parallelism.

    x [T, H] → router (top-k of E) → dispatch (put + signal over NVLink) → per-expert SwiGLU MLP on the
    grouped tcgen05 GEMM → combine (put + signal) → weighted sum → y [T, H]

A thin, named configuration of ``ops.moe.MoELayer`` (hidden 4096, FFN 14336, 8 experts, top-2 are
Mixtral-8x7B's) plus the autograd bridge.  The reference has no model code; dispatch/combine are built on
this package's device-side put-with-signal (OpenSHMEM 1.5 semantics).
"""
from __future__ import annotations

import torch

from ..ops.moe import MoELayer, interleave_gate_up


class MixtralMoEBlock(MoELayer):
    def __init__(self, rt, hidden: int = 4096, ffn: int = 14336, n_experts: int = 8, topk: int = 2, max_tokens: int = 16384,
                 capacity_factor: float = 1.25, training: bool = True, timeout_ms: int = 4000):
        super().__init__(rt, hidden, ffn, n_experts, topk, max_tokens, capacity_factor=capacity_factor, training=training,
                         timeout_ms=timeout_ms)

    def load(self, w_router: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> None:
        """w_router [E, H]; this rank's experts: w_gate / w_up [E/P, F, H], w_down [E/P, H, F]."""
        self.wr.copy_(w_router)
        self.w2.copy_(w_down)
        for g in range(self.G):
            self.w13[g].copy_(interleave_gate_up(w_gate[g].to(torch.bfloat16), w_up[g].to(torch.bfloat16)))
        self.sync_transposes()


class _MoEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w13, w2, wr, block):
        ctx.block = block
        return block.forward(x).clone()

    @staticmethod
    def backward(ctx, dy):
        block = ctx.block
        dx = block.backward(dy.contiguous())
        return dx.clone(), block.dw13.clone(), block.dw2.clone(), block.dwr.clone(), None


class MixtralMoEModule(torch.nn.Module):
    """``torch.nn.Module`` face: expert and router weights are parameters aliasing the block's buffers; the backward
    pass returns gradients for all of them and for the input (expert path plus the path through the router's
    softmax over the chosen experts)."""

    def __init__(self, rt, **kw):
        super().__init__()
        self.block = MixtralMoEBlock(rt, training=True, **kw)
        self.w13 = torch.nn.Parameter(self.block.w13)
        self.w2 = torch.nn.Parameter(self.block.w2)
        self.wr = torch.nn.Parameter(self.block.wr)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return _MoEFn.apply(x, self.w13, self.w2, self.wr, self.block)

    def after_step(self) -> None:
        self.block.sync_transposes()
