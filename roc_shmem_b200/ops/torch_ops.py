"""PyTorch operator registration for the hand-written kernels.

``torch.ops.bshmem.linear(x, w)`` is ``x @ w.T`` on the tcgen05 GEMM with a registered fake (meta)
implementation and an autograd formula whose two gradients also run on the tcgen05 kernels
(data gradient: K-major GEMM on a transposed weight copy; weight gradient: the transposed-operand
MN-major GEMM, no activation transpose).  ``torch.ops.bshmem.linear_fp8`` quantises both operands
to block-scaled e4m3 and runs the fp8 kernel (forward only).  The reference has no PyTorch layer.
"""
from __future__ import annotations

import torch

from .gemm import gemm_bf16
from .gemm_fp8 import gemm_fp8, quantize_act, quantize_weight


def _check_linear(x: torch.Tensor, w: torch.Tensor) -> None:
    if x.dim() != 2 or w.dim() != 2 or x.shape[1] != w.shape[1]:
        raise ValueError(f"linear: shape mismatch {tuple(x.shape)} x {tuple(w.shape)}")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise ValueError("linear: bf16 operands only")


@torch.library.custom_op("bshmem::linear", mutates_args=())
def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    _check_linear(x, w)
    return gemm_bf16(x.contiguous(), w.contiguous())


@linear.register_fake
def _(x, w):
    return x.new_empty((x.shape[0], w.shape[0]))


@torch.library.custom_op("bshmem::linear_wgrad", mutates_args=())
def linear_wgrad(dy: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """dW[N, K] = dy[M, N].T @ x[M, K] on token-major operands (needs M % 64 == 0, N % 256 == 0, K % 256 == 0;
    other shapes fall back to transposing dy and x once and using the K-major kernel)."""
    from .moe import grouped_gemm_tn
    M, N = dy.shape
    K = x.shape[1]
    out = torch.empty((N, K), dtype=torch.bfloat16, device=x.device)
    if M % 64 == 0 and N % 256 == 0 and K % 256 == 0:
        rows = torch.full((1,), M, dtype=torch.int32, device=x.device)
        grouped_gemm_tn(dy.contiguous(), x.contiguous(), out, 1, rows)
        return out
    if M % 8:
        raise ValueError("linear_wgrad: the token count must be a multiple of 8")
    return gemm_bf16(dy.t().contiguous(), x.t().contiguous(), out)


@linear_wgrad.register_fake
def _(dy, x):
    return x.new_empty((dy.shape[1], x.shape[1]))


def _linear_setup(ctx, inputs, output):
    ctx.save_for_backward(*inputs)


def _linear_backward(ctx, dy):
    x, w = ctx.saved_tensors
    dy = dy.contiguous()
    dx = torch.ops.bshmem.linear(dy, w.t().contiguous()) if ctx.needs_input_grad[0] else None
    dw = torch.ops.bshmem.linear_wgrad(dy, x) if ctx.needs_input_grad[1] else None
    return dx, dw


linear.register_autograd(_linear_backward, setup_context=_linear_setup)


@torch.library.custom_op("bshmem::linear_fp8", mutates_args=())
def linear_fp8(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x @ w.T with both operands quantised on the fly to block-scaled e4m3 (1x128 / 128x128 scales)."""
    _check_linear(x, w)
    return gemm_fp8(quantize_act(x.contiguous()), quantize_weight(w.contiguous()))


@linear_fp8.register_fake
def _(x, w):
    return x.new_empty((x.shape[0], w.shape[0]))


class Linear(torch.nn.Module):
    """Drop-in bf16 ``nn.Linear`` (no bias) whose forward and both gradients run on the tcgen05 kernels."""

    def __init__(self, in_features: int, out_features: int, device=None):
        super().__init__()
        self.weight = torch.nn.Parameter(torch.empty((out_features, in_features), dtype=torch.bfloat16, device=device))
        torch.nn.init.normal_(self.weight, std=0.02)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        y = torch.ops.bshmem.linear(x.reshape(-1, x.shape[-1]), self.weight)
        return y.reshape(*lead, -1)


# ---- collectives on the calling PE's runtime (roc_shmem_b200.current()) --------------------------------
# Arbitrary tensors are staged through symmetric scratch that is cached per (shape, dtype); symmetric
# tensors (rt.empty / rt.zeros) are used in place.  Works on the NVLink and on the CPU backend.
_scratch: dict = {}


def _sym(rt, key: str, shape, dtype) -> torch.Tensor:
    k = (id(rt), key, tuple(shape), dtype)
    t = _scratch.get(k)
    if t is None:
        t = rt.empty(tuple(shape), dtype)
        _scratch[k] = t
    return t


def release_scratch() -> None:
    """Free the cached symmetric staging buffers (collective: every PE must call it)."""
    from .. import current
    rt = current()
    for k in [k for k in _scratch if k[0] == id(rt)]:
        rt.free(_scratch.pop(k))


@torch.library.custom_op("bshmem::all_reduce", mutates_args=())
def all_reduce(x: torch.Tensor, op: str = "sum") -> torch.Tensor:
    """Reduction over all PEs (`to_all`); every PE gets the result."""
    from .. import current
    rt = current()
    src, dst = _sym(rt, "ar_src", x.shape, x.dtype), _sym(rt, "ar_dst", x.shape, x.dtype)
    src.copy_(x)
    rt.reduce(dst, src, op)
    return dst.clone()


@all_reduce.register_fake
def _(x, op="sum"):
    return torch.empty_like(x)


@torch.library.custom_op("bshmem::all_gather", mutates_args=())
def all_gather(x: torch.Tensor) -> torch.Tensor:
    """Concatenation of every PE's `x` along dimension 0 (`fcollect`)."""
    from .. import current
    rt = current()
    src = _sym(rt, "ag_src", x.shape, x.dtype)
    dst = _sym(rt, "ag_dst", (rt.n_pes * x.shape[0],) + tuple(x.shape[1:]), x.dtype)
    src.copy_(x)
    rt.fcollect(dst, src)
    return dst.clone()


@all_gather.register_fake
def _(x):
    from .. import current
    return x.new_empty((current().n_pes * x.shape[0],) + tuple(x.shape[1:]))


@torch.library.custom_op("bshmem::reduce_scatter", mutates_args=())
def reduce_scatter(x: torch.Tensor, op: str = "sum") -> torch.Tensor:
    """This PE's 1/n slice (dimension 0) of the reduction of every PE's `x`."""
    from .. import current
    rt = current()
    if x.shape[0] % rt.n_pes:
        raise ValueError("reduce_scatter: dimension 0 must divide by the number of PEs")
    src = _sym(rt, "rs_src", x.shape, x.dtype)
    dst = _sym(rt, "rs_dst", (x.shape[0] // rt.n_pes,) + tuple(x.shape[1:]), x.dtype)
    src.copy_(x)
    rt.reduce_scatter(dst, src, op)
    return dst.clone()


@reduce_scatter.register_fake
def _(x, op="sum"):
    from .. import current
    return x.new_empty((x.shape[0] // current().n_pes,) + tuple(x.shape[1:]))


@torch.library.custom_op("bshmem::all_to_all", mutates_args=())
def all_to_all(x: torch.Tensor) -> torch.Tensor:
    """Block k (dimension 0 split in n equal blocks) of PE j's `x` becomes block j of PE k's result."""
    from .. import current
    rt = current()
    if x.shape[0] % rt.n_pes:
        raise ValueError("all_to_all: dimension 0 must divide by the number of PEs")
    src, dst = _sym(rt, "a2a_src", x.shape, x.dtype), _sym(rt, "a2a_dst", x.shape, x.dtype)
    src.copy_(x)
    rt.alltoall(dst, src)
    return dst.clone()


@all_to_all.register_fake
def _(x):
    return torch.empty_like(x)


def _ar_backward(ctx, g):
    return torch.ops.bshmem.all_reduce(g.contiguous(), "sum"), None


def _ag_backward(ctx, g):
    return torch.ops.bshmem.reduce_scatter(g.contiguous(), "sum")


def _rs_backward(ctx, g):
    return torch.ops.bshmem.all_gather(g.contiguous()), None


def _a2a_backward(ctx, g):
    return torch.ops.bshmem.all_to_all(g.contiguous())


# gradients of the sum-collectives are the matching collectives (valid for op == "sum")
all_reduce.register_autograd(_ar_backward)
all_gather.register_autograd(_ag_backward)
reduce_scatter.register_autograd(_rs_backward)
all_to_all.register_autograd(_a2a_backward)
