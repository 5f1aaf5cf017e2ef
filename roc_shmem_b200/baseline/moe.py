"""Baseline MoE layer: NCCL all_to_all_single for dispatch / combine and cuBLAS (torch.matmul)
for the expert FFN, with autograd for the backward pass.  Used for the correctness oracle
(fp32 mode) and as the timing baseline (bf16 mode).  A path that only calls NCCL is the
baseline, not the product."""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as Fn


def route(x: torch.Tensor, wr: torch.Tensor, topk: int):
    probs = torch.softmax(x.float() @ wr.float().t(), dim=-1)
    w, idx = torch.topk(probs, topk, dim=-1)          # ties: lower index first, like the kernel
    w = w / w.sum(-1, keepdim=True)
    return idx, w


def expert_ffn(xe: torch.Tensor, w1: torch.Tensor, w3: torch.Tensor, w2: torch.Tensor) -> torch.Tensor:
    return (Fn.silu(xe @ w1.t()) * (xe @ w3.t())) @ w2.t()


def moe_reference_single(x, wr, w1, w3, w2, topk, compute_dtype=torch.float32, router_grad=False):
    """All experts local (no communication): plain PyTorch, differentiable.  w1/w3: [E, F, H], w2: [E, H, F].
    With `router_grad` the routing weights stay in the autograd graph (gradients reach `wr` and, through the router, `x`)."""
    idx, w = route(x if router_grad else x.detach(), wr, topk)
    out = torch.zeros(x.shape, dtype=compute_dtype, device=x.device)
    xc = x.to(compute_dtype)
    for e in range(w1.shape[0]):
        tok, k = (idx == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        ye = expert_ffn(xc[tok], w1[e].to(compute_dtype), w3[e].to(compute_dtype), w2[e].to(compute_dtype))
        out.index_add_(0, tok, ye * w[tok, k].to(compute_dtype).unsqueeze(-1))
    return out, idx, w


class NcclMoE(torch.nn.Module):
    """Expert-parallel MoE with NCCL all_to_all and cuBLAS, one expert group per rank."""

    def __init__(self, wr, w1, w3, w2, topk: int, router_grad: bool = False):
        """With `router_grad` the routing weights stay in the autograd graph: backward also yields the router weight
        gradient and the router's share of the input gradient (what MoELayer.backward computes)."""
        super().__init__()
        self.router_grad = router_grad
        self.wr = torch.nn.Parameter(wr.clone()) if router_grad else wr
        self.w1 = torch.nn.Parameter(w1)      # [G, F, H] local experts
        self.w3 = torch.nn.Parameter(w3)
        self.w2 = torch.nn.Parameter(w2)      # [G, H, F]
        self.topk = topk

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        P = dist.get_world_size() if dist.is_initialized() else 1
        G = self.w1.shape[0]
        E = G * P
        T, H = x.shape
        idx, w = route(x if self.router_grad else x.detach(), self.wr, self.topk)
        flat_e = idx.reshape(-1)
        order = torch.argsort(flat_e, stable=True)
        tok = order // self.topk
        send = x[tok]                                            # rows sorted by destination expert
        counts = torch.bincount(flat_e, minlength=E)
        if P > 1:
            recv_counts = torch.empty_like(counts)
            dist.all_to_all_single(recv_counts, counts)          # [P * G]: rows per (source rank, local expert)
            in_splits = counts.view(P, G).sum(1).tolist()
            out_splits = recv_counts.view(P, G).sum(1).tolist()
            recv = _AllToAll.apply(send, out_splits, in_splits)
            rc = recv_counts.view(P, G)
        else:
            recv, rc = send, counts.view(1, G)
        # rows arrive grouped by source rank then expert: regroup per expert
        pieces = recv.split(rc.reshape(-1).tolist())
        outs = [None] * len(pieces)
        for g in range(G):
            rows = torch.cat([pieces[s * G + g] for s in range(P)]) if P > 1 else pieces[g]
            ye = expert_ffn(rows, self.w1[g], self.w3[g], self.w2[g])
            for s, part in zip(range(P), ye.split([int(rc[s, g]) for s in range(P)])):
                outs[s * G + g] = part
        back = torch.cat(outs)
        if P > 1:
            back = _AllToAll.apply(back, in_splits, out_splits)
        y = torch.zeros_like(x)
        y.index_add_(0, tok, back * w.reshape(-1)[order].to(back.dtype).unsqueeze(-1))
        return y


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_splits, in_splits):
        ctx.out_splits, ctx.in_splits = out_splits, in_splits
        out = x.new_empty((sum(out_splits),) + x.shape[1:])
        dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits)
        return out

    @staticmethod
    def backward(ctx, g):
        out = g.new_empty((sum(ctx.in_splits),) + g.shape[1:])
        dist.all_to_all_single(out, g.contiguous(), ctx.in_splits, ctx.out_splits)
        return out, None, None
