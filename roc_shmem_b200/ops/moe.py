"""Expert-parallel MoE layer on the device API: router, dispatch / combine over NVLink
with put + signal semantics, grouped tcgen05 expert GEMMs, forward and backward.

Mixtral-style: E experts spread over P PEs (E/P per PE), top-k routing with softmax
over all experts and renormalisation over the chosen ones, SwiGLU experts
(w1 = gate, w3 = up, w2 = down).  The kernels are in csrc/cuda/moe_kernels.cu and
moe_gemm.cu; the NCCL all_to_all + cuBLAS equivalent is roc_shmem_b200/baseline/moe.py.
The reference has no MoE layer — this is a north-star workload built on its device API
shape (put, signal, wait).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from .. import _native
from ..gpu import DevState

_declared = False
SIG_FWD_DISPATCH, SIG_FWD_COMBINE, SIG_BWD_DISPATCH, SIG_BWD_COMBINE = range(4)


class PlanDev(C.Structure):
    """Mirror of MoePlanDev."""
    _fields_ = [("P", C.c_int), ("E", C.c_int), ("me", C.c_int), ("cap", C.c_int), ("base_me", C.c_void_p),
                ("src_start", C.c_void_p), ("recv_count", C.c_void_p), ("expect_from", C.c_void_p), ("send_to", C.c_void_p),
                ("dropped", C.c_void_p), ("arrive_sig", C.c_void_p)]


def moe_lib() -> C.CDLL:
    global _declared
    lib = _native.load("libbshmem_moe.so")
    if not _declared:
        VP, I = C.c_void_p, C.c_int
        PS, PP = C.POINTER(DevState), C.POINTER(PlanDev)

        def f(name, *args, res=I):
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, list(args)
        f("bshmem_moe_last_error", res=C.c_char_p)
        f("bshmem_moe_gemm_last_error", res=C.c_char_p)
        f("bshmem_moe_router_topk", VP, VP, I, I, I, I, VP, VP, VP, VP)
        f("bshmem_moe_plan", VP, I, I, VP, VP, VP)
        f("bshmem_moe_offsets", PP, VP, I, VP)
        f("bshmem_moe_dispatch", PS, PP, VP, VP, VP, VP, I, I, I, VP, VP, I, I, I, VP)
        f("bshmem_moe_wait_arrivals", PP, I, I, VP, I, VP, VP)
        f("bshmem_moe_combine_send", PS, PP, VP, VP, I, VP, I, I, I, VP)
        f("bshmem_moe_combine_reduce", PP, VP, VP, VP, VP, I, I, I, VP, VP)
        f("bshmem_moe_router_weight_grad", PP, VP, VP, VP, VP, I, I, I, VP, VP)
        f("bshmem_moe_router_backward", VP, VP, VP, VP, I, I, I, I, VP, VP, VP, VP)
        f("bshmem_moe_combine_reduce_router", PP, VP, VP, VP, I, I, I, VP, VP, VP, VP)
        f("bshmem_moe_swiglu_fwd", VP, VP, I, I, I, VP, VP)
        f("bshmem_moe_swiglu_bwd", VP, VP, VP, I, I, I, VP, VP)
        f("bshmem_moe_transpose_pad", VP, VP, I, I, I, VP, VP)
        f("bshmem_moe_grouped_gemm", VP, VP, VP, I, I, I, I, I, I, I, I, VP, I, VP, I, VP, VP, I, VP, I, I)
        f("bshmem_moe_grouped_gemm_tn", VP, VP, VP, I, I, I, I, I, I, I, VP, VP, I, I)
        f("bshmem_moe_zero_pad_rows", VP, VP, I, I, I, VP)
        f("bshmem_moe_gemm_error_site", I)
        f("bshmem_moe_gemm_error_word", res=VP)
        _declared = True
    return lib


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


def interleave_gate_up(w1: torch.Tensor, w3: torch.Tensor) -> torch.Tensor:
    """[F, H] gate and [F, H] up weights → [2F, H] with 32 gate rows followed by the matching 32 up rows,
    the layout the gated epilogue and the SwiGLU kernels expect."""
    F, H = w1.shape
    assert F % 32 == 0 and w3.shape == w1.shape
    return torch.stack((w1.view(F // 32, 32, H), w3.view(F // 32, 32, H)), dim=1).reshape(2 * F, H).contiguous()


def grouped_gemm(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, groups: int, *, rows: Optional[torch.Tensor] = None,
                 fixed_rows: int = 0, klen: Optional[torch.Tensor] = None, gated: bool = False, arrive=None, expected=None,
                 n_arrive: int = 0, timeout_ms: int = 4000, max_ctas: int = 0) -> None:
    """out_g = a_g @ b_g.T per group on the tcgen05 grouped kernel.  a: [G*Ra, K], b: [G*Rb, K], out: [G*Ra, N or N/2]."""
    lib = moe_lib()
    G = groups
    ra, rb = a.shape[0] // G, b.shape[0] // G
    K = a.shape[1]
    N = rb
    st = lib.bshmem_moe_grouped_gemm(a.data_ptr(), b.data_ptr(), out.data_ptr(), G, ra, rb, N, K, a.stride(0), b.stride(0),
                                     out.stride(0), _p(rows), fixed_rows, _p(klen), int(gated), arrive or 0, _p(expected),
                                     n_arrive, _stream(), timeout_ms, max_ctas)
    if st != 0:
        raise RuntimeError(f"grouped gemm failed ({st}): {lib.bshmem_moe_gemm_last_error().decode()}")


def grouped_gemm_tn(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, groups: int, counts: torch.Tensor, *,
                    timeout_ms: int = 4000, max_ctas: int = 0) -> None:
    """out_g[M, N] = a_g.T @ b_g per group with token-major operands a: [G*cap, M], b: [G*cap, N] and
    `counts[g]` tokens per group; both operands go to the tensor core MN-major, no transpose is materialised.
    Token rows [counts[g], next multiple of 64) of a and b must be zero (see zero_pad_rows)."""
    lib = moe_lib()
    G = groups
    cap = a.shape[0] // G
    st = lib.bshmem_moe_grouped_gemm_tn(a.data_ptr(), b.data_ptr(), out.data_ptr(), G, cap, a.shape[1], b.shape[1], a.stride(0),
                                        b.stride(0), out.stride(0), counts.data_ptr(), _stream(), timeout_ms, max_ctas)
    if st != 0:
        raise RuntimeError(f"grouped gemm (tn) failed ({st}): {lib.bshmem_moe_gemm_last_error().decode()}")


def zero_pad_rows(buf: torch.Tensor, groups: int, counts: torch.Tensor) -> None:
    """Zero rows [counts[g], next multiple of 64) of every group of a contiguous [G*cap, cols] bf16 buffer."""
    lib = moe_lib()
    assert buf.is_contiguous()
    st = lib.bshmem_moe_zero_pad_rows(buf.data_ptr(), counts.data_ptr(), groups, buf.shape[0] // groups, buf.shape[1], _stream())
    if st != 0:
        raise RuntimeError(f"zero_pad_rows failed ({st}): {lib.bshmem_moe_gemm_last_error().decode()}")


class MoELayer:
    """One MoE block: y[T, H] = combine(experts(dispatch(x)))  with forward and backward.

    Weights per local expert: `w13` [G, 2F, H] (interleaved gate/up, see interleave_gate_up), `w2` [G, H, F];
    router `wr` [E, H].  Transposed copies used by the backward data-gradient GEMMs are kept in sync by
    `sync_transposes()` (all operands of the tcgen05 kernels are K-major)."""

    def __init__(self, rt, hidden: int, ffn: int, n_experts: int, topk: int, max_tokens: int, capacity_factor: float = 1.25,
                 training: bool = True, timeout_ms: int = 4000, tn_gemm: bool = True):
        self.tn_gemm = tn_gemm          # weight gradients on MN-major operands (False: explicit transposes)
        self.rt, self.H, self.F, self.E, self.topk, self.T = rt, hidden, ffn, n_experts, topk, max_tokens
        self.lib = moe_lib()
        P = rt.n_pes
        assert n_experts % P == 0 and hidden % 256 == 0 and ffn % 256 == 0
        self.P, self.G = P, n_experts // P
        cap = int(max_tokens * topk * P / n_experts * capacity_factor)
        self.cap = (cap + 255) // 256 * 256
        self.training, self.timeout_ms = training, timeout_ms
        dev, bf = rt.device, torch.bfloat16
        G, cap, H, F, T = self.G, self.cap, hidden, ffn, max_tokens
        n_entries = T * topk
        # ---- weights (random init by the caller) ----
        self.wr = torch.empty((n_experts, H), dtype=bf, device=dev)
        self.w13 = torch.empty((G, 2 * F, H), dtype=bf, device=dev)
        self.w2 = torch.empty((G, H, F), dtype=bf, device=dev)
        # ---- routing state ----
        self.topk_idx = torch.empty((n_entries,), dtype=torch.int32, device=dev)
        self.topk_w = torch.empty((n_entries,), dtype=torch.float32, device=dev)
        self.pos = torch.empty((n_entries,), dtype=torch.int32, device=dev)
        self.counts = rt.zeros((n_experts,), torch.int32)                     # symmetric: gathered below
        self.counts_all = rt.zeros((P * n_experts,), torch.int32)
        self.base_me = torch.zeros((n_experts,), dtype=torch.int32, device=dev)
        self.src_start = torch.zeros((G * (P + 1),), dtype=torch.int32, device=dev)
        self.recv_count = torch.zeros((G,), dtype=torch.int32, device=dev)
        self.expect_from = torch.zeros((P,), dtype=torch.int32, device=dev)
        self.send_to = torch.zeros((P,), dtype=torch.int32, device=dev)
        self.dropped = torch.zeros((1,), dtype=torch.int32, device=dev)
        self.arrive = rt.zeros((2 * 4 * P,), torch.int64)
        # ---- symmetric data buffers ----
        self.recv = rt.empty((G * cap, H), bf, align=1024)                    # dispatched tokens (kept for dW13 in training)
        self.meta = rt.empty((G * cap,), torch.int32)
        self.ybuf = rt.empty((n_entries, H), bf, align=1024)                  # expert outputs per entry, back at the source
        # ---- expert-side activations ----
        self.gu = torch.empty((G * cap, 2 * F), dtype=bf, device=dev)
        self.hact = torch.empty((G * cap, F), dtype=bf, device=dev)
        self.yexp = torch.empty((G * cap, H), dtype=bf, device=dev)
        self.out = torch.empty((T, H), dtype=bf, device=dev)
        if training:
            # the backward pass dispatches gradients into a receive buffer of its own, so the forward's dispatched
            # inputs stay where they landed until dW13 has read them (no copy)
            self.recv_bwd = rt.empty((G * cap, H), bf, align=1024)
            self.xsave = self.recv
            self.w13_t = torch.empty((G, H, 2 * F), dtype=bf, device=dev)
            self.w2_t = torch.empty((G, F, H), dtype=bf, device=dev)
            self.dh = torch.empty((G * cap, F), dtype=bf, device=dev)
            self.dgu = torch.empty((G * cap, 2 * F), dtype=bf, device=dev)
            self.dxe = torch.empty((G * cap, H), dtype=bf, device=dev)
            if not tn_gemm:
                self.t_a = torch.empty((G * 2 * F * cap,), dtype=bf, device=dev)  # transposed operands, reused
                self.t_b = torch.empty((G * max(F, H) * cap,), dtype=bf, device=dev)
            self.dw13 = torch.empty((G, 2 * F, H), dtype=bf, device=dev)
            self.dw2 = torch.empty((G, H, F), dtype=bf, device=dev)
            self.dxbuf = rt.empty((n_entries, H), bf, align=1024)
            self.dx = torch.empty((T, H), dtype=bf, device=dev)
            self.dtopk_w = torch.empty((n_entries,), dtype=torch.float32, device=dev)
            self.dlogit = torch.empty((n_entries,), dtype=torch.float32, device=dev)   # gradient of the chosen experts' logits
            self.dwr_f32 = torch.empty((n_experts, H), dtype=torch.float32, device=dev)
            self.dwr = torch.empty((n_experts, H), dtype=bf, device=dev)             # router weight gradient
            self._x_in = None
        self.plan = PlanDev(P=P, E=n_experts, me=rt.my_pe, cap=self.cap, base_me=self.base_me.data_ptr(),
                            src_start=self.src_start.data_ptr(), recv_count=self.recv_count.data_ptr(),
                            expect_from=self.expect_from.data_ptr(), send_to=self.send_to.data_ptr(),
                            dropped=self.dropped.data_ptr(), arrive_sig=self.arrive.data_ptr())
        self.state = rt.device_state()
        self.err_word = self.lib.bshmem_moe_gemm_error_word()
        self.calls = 0
        self.launches = 0
        self.ctas = 128
        rt.barrier_all()

    # ------------------------------------------------------------------------------------
    def sync_transposes(self) -> None:
        """Refresh the transposed weight copies the backward data-gradient GEMMs read."""
        if self.training:
            self.w13_t.copy_(self.w13.transpose(1, 2))
            self.w2_t.copy_(self.w2.transpose(1, 2))

    def _chk(self, st: int, what: str) -> None:
        if st != 0:
            raise RuntimeError(f"{what} failed ({st}): {self.lib.bshmem_moe_last_error().decode()}")
        self.launches += 1

    def _sig_ptr(self, parity: int, which: int) -> int:
        return self.arrive.data_ptr() + 8 * (parity * 4 * self.P + which * self.P)

    def route(self, x: torch.Tensor) -> None:
        """Router, plan, count exchange and offsets for this call's tokens."""
        lib, T, s = self.lib, x.shape[0], _stream()
        n_entries = T * self.topk
        self.calls += 1
        self.parity = self.calls & 1
        self._chk(lib.bshmem_moe_router_topk(x.data_ptr(), self.wr.data_ptr(), T, self.H, self.E, self.topk,
                                             self.topk_idx.data_ptr(), self.topk_w.data_ptr(), 0, s), "router")
        self._chk(lib.bshmem_moe_plan(self.topk_idx.data_ptr(), n_entries, self.E, self.pos.data_ptr(),
                                      self.counts.data_ptr(), s), "plan")
        if self.P > 1:
            self.rt.fcollect(self.counts_all, self.counts)        # all-gather of the per-expert counts (device collective)
            self.launches += 1
        else:
            self.counts_all.copy_(self.counts)
        self._chk(lib.bshmem_moe_offsets(C.byref(self.plan), self.counts_all.data_ptr(), self.parity, s), "offsets")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lib, T, s = self.lib, x.shape[0], _stream()
        n_entries = T * self.topk
        G, cap, H, F, P = self.G, self.cap, self.H, self.F, self.P
        self.route(x)
        par = self.parity
        self._chk(lib.bshmem_moe_dispatch(C.byref(self.state), C.byref(self.plan), x.data_ptr(), 0, self.topk_idx.data_ptr(),
                                          self.pos.data_ptr(), n_entries, self.topk, H, self.recv.data_ptr(), self.meta.data_ptr(),
                                          par, SIG_FWD_DISPATCH, self.ctas, s), "dispatch")
        # gate/up projection waits on the arrival words inside the kernel, then SwiGLU, then down projection
        if self.training:
            grouped_gemm(self.recv, self.w13.view(G * 2 * F, H), self.gu, G, rows=self.recv_count,
                         arrive=self._sig_ptr(par, SIG_FWD_DISPATCH), expected=self.expect_from, n_arrive=P,
                         timeout_ms=self.timeout_ms)
            self._chk(lib.bshmem_moe_swiglu_fwd(self.gu.data_ptr(), self.recv_count.data_ptr(), G, cap, F, self.hact.data_ptr(), s),
                      "swiglu")
            self._x_in = x                                         # the router's backward needs the layer input
        else:
            grouped_gemm(self.recv, self.w13.view(G * 2 * F, H), self.hact, G, rows=self.recv_count, gated=True,
                         arrive=self._sig_ptr(par, SIG_FWD_DISPATCH), expected=self.expect_from, n_arrive=P,
                         timeout_ms=self.timeout_ms)
        self.launches += 1
        grouped_gemm(self.hact, self.w2.view(G * H, F), self.yexp, G, rows=self.recv_count, timeout_ms=self.timeout_ms)
        self.launches += 1
        self._chk(lib.bshmem_moe_combine_send(C.byref(self.state), C.byref(self.plan), self.yexp.data_ptr(), self.meta.data_ptr(), H,
                                              self.ybuf.data_ptr(), par, SIG_FWD_COMBINE, self.ctas, s), "combine_send")
        self._chk(lib.bshmem_moe_wait_arrivals(C.byref(self.plan), par, SIG_FWD_COMBINE, self.send_to.data_ptr(), self.timeout_ms,
                                               self.err_word, s), "wait")
        self._chk(lib.bshmem_moe_combine_reduce(C.byref(self.plan), self.ybuf.data_ptr(), self.topk_w.data_ptr(),
                                                self.topk_idx.data_ptr(), self.pos.data_ptr(), T, self.topk, H, self.out.data_ptr(), s),
                  "combine_reduce")
        return self.out[:T]

    def backward(self, dout: torch.Tensor) -> torch.Tensor:
        """Gradients w.r.t. the layer input (returned; expert path and router path), the expert weights (self.dw13,
        self.dw2), the routing weights (self.dtopk_w) and, through the softmax over the chosen experts, the router
        weights (self.dwr).  Must follow forward() of the same tokens; the forward's input must still be intact."""
        assert self.training
        lib, T, s = self.lib, dout.shape[0], _stream()
        n_entries = T * self.topk
        G, cap, H, F, P = self.G, self.cap, self.H, self.F, self.P
        par = self.parity
        rc = self.recv_count
        self._chk(lib.bshmem_moe_router_weight_grad(C.byref(self.plan), self.ybuf.data_ptr(), dout.data_ptr(),
                                                    self.topk_idx.data_ptr(), self.pos.data_ptr(), n_entries, self.topk, H,
                                                    self.dtopk_w.data_ptr(), s), "router weight grad")
        # router backward: d_logits of the chosen experts and d_Wr = d_logits^T · x
        self._chk(lib.bshmem_moe_router_backward(self._x_in.data_ptr(), self.topk_idx.data_ptr(), self.topk_w.data_ptr(),
                                                 self.dtopk_w.data_ptr(), T, H, self.E, self.topk, self.dlogit.data_ptr(),
                                                 self.dwr_f32.data_ptr(), self.dwr.data_ptr(), s), "router backward")
        self.launches += 2
        # combine-backward = dispatch of w * d_out into the experts' gradient receive buffers (same slots as forward)
        dy = self.recv_bwd
        self._chk(lib.bshmem_moe_dispatch(C.byref(self.state), C.byref(self.plan), dout.data_ptr(), self.topk_w.data_ptr(),
                                          self.topk_idx.data_ptr(), self.pos.data_ptr(), n_entries, self.topk, H, dy.data_ptr(),
                                          0, par, SIG_BWD_DISPATCH, self.ctas, s), "dispatch(bwd)")
        # d_hact = d_y · W2            (B operand = W2^T [F, H], K = H)
        grouped_gemm(dy, self.w2_t.view(G * F, H), self.dh, G, rows=rc, arrive=self._sig_ptr(par, SIG_BWD_DISPATCH),
                     expected=self.expect_from, n_arrive=P, timeout_ms=self.timeout_ms)
        # dW2 = d_y^T · hact: token-major operands straight into the MN-major tensor-core path
        if self.tn_gemm:
            zero_pad_rows(dy, G, rc)
            zero_pad_rows(self.hact, G, rc)
            grouped_gemm_tn(dy, self.hact, self.dw2.view(G * H, F), G, rc, timeout_ms=self.timeout_ms)
        else:                          # explicit transposes + ragged-K K-major GEMM
            ta = self.t_a[: G * H * cap].view(G * H, cap)
            tb = self.t_b[: G * F * cap].view(G * F, cap)
            self._chk(lib.bshmem_moe_transpose_pad(dy.data_ptr(), rc.data_ptr(), G, cap, H, ta.data_ptr(), s), "transpose")
            self._chk(lib.bshmem_moe_transpose_pad(self.hact.data_ptr(), rc.data_ptr(), G, cap, F, tb.data_ptr(), s), "transpose")
            grouped_gemm(ta, tb, self.dw2.view(G * H, F), G, fixed_rows=H, klen=rc, timeout_ms=self.timeout_ms)
        # SwiGLU backward, then dW13 = d_gu^T · x and d_x = d_gu · W13
        self._chk(lib.bshmem_moe_swiglu_bwd(self.gu.data_ptr(), self.dh.data_ptr(), rc.data_ptr(), G, cap, F, self.dgu.data_ptr(), s),
                  "swiglu bwd")
        if self.tn_gemm:
            zero_pad_rows(self.dgu, G, rc)
            zero_pad_rows(self.xsave, G, rc)
            grouped_gemm_tn(self.dgu, self.xsave, self.dw13.view(G * 2 * F, H), G, rc, timeout_ms=self.timeout_ms)
        else:
            ta2 = self.t_a[: G * 2 * F * cap].view(G * 2 * F, cap)
            tb2 = self.t_b[: G * H * cap].view(G * H, cap)
            self._chk(lib.bshmem_moe_transpose_pad(self.dgu.data_ptr(), rc.data_ptr(), G, cap, 2 * F, ta2.data_ptr(), s), "transpose")
            self._chk(lib.bshmem_moe_transpose_pad(self.xsave.data_ptr(), rc.data_ptr(), G, cap, H, tb2.data_ptr(), s), "transpose")
            grouped_gemm(ta2, tb2, self.dw13.view(G * 2 * F, H), G, fixed_rows=2 * F, klen=rc, timeout_ms=self.timeout_ms)
        grouped_gemm(self.dgu, self.w13_t.view(G * H, 2 * F), self.dxe, G, rows=rc, timeout_ms=self.timeout_ms)
        self.launches += 4
        # dispatch-backward = combine of the d_x rows back to their source entries, summed over k
        self._chk(lib.bshmem_moe_combine_send(C.byref(self.state), C.byref(self.plan), self.dxe.data_ptr(), self.meta.data_ptr(), H,
                                              self.dxbuf.data_ptr(), par, SIG_BWD_COMBINE, self.ctas, s), "combine_send(bwd)")
        self._chk(lib.bshmem_moe_wait_arrivals(C.byref(self.plan), par, SIG_BWD_COMBINE, self.send_to.data_ptr(), self.timeout_ms,
                                               self.err_word, s), "wait")
        # d_x = sum over k of the returned rows + the router path (d_logits · Wr), written once
        self._chk(lib.bshmem_moe_combine_reduce_router(C.byref(self.plan), self.dxbuf.data_ptr(), self.topk_idx.data_ptr(),
                                                       self.pos.data_ptr(), T, self.topk, H, self.dx.data_ptr(),
                                                       self.dlogit.data_ptr(), self.wr.data_ptr(), s), "combine_reduce(bwd)")
        return self.dx[:T]

    def check(self) -> None:
        site = self.lib.bshmem_moe_gemm_error_site(1)
        if site:
            raise RuntimeError(f"moe: a bounded in-kernel wait ran out (site {site})")
        if int(self.dropped.item()):
            raise RuntimeError(f"moe: {int(self.dropped.item())} rows exceeded the expert capacity {self.cap}")
