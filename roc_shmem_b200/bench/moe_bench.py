"""MoE expert-parallel layer: device-API dispatch/combine + grouped tcgen05 GEMMs versus
NCCL all_to_all + cuBLAS, forward + backward, device-timed (max over ranks).

    torchrun --nproc-per-node P -m roc_shmem_b200.bench.moe_bench [--small] [--iters 5] [--out file.json]

Config: Mixtral-style, 8 experts, top-2, hidden 4096, expert ffn 14336 (SwiGLU), 16384 tokens per
rank, bf16; router logits from N(0,1) activations and weights, expert weights N(0,0.02).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

import roc_shmem_b200 as shmem
from roc_shmem_b200.baseline.moe import NcclMoE
from roc_shmem_b200.ops.moe import MoELayer, interleave_gate_up


def timed(fn, iters, rt):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    rt.barrier_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    if dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--mid", action="store_true", help="4096 tokens, hidden 2048, ffn 4096 (profiler captures)")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--out", default="")
    ap.add_argument("--no-baseline", action="store_true")
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--topk", type=int, default=2)
    args = ap.parse_args()
    rank, P = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    for k, v in (("RANK", "0"), ("WORLD_SIZE", "1"), ("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", "29533")):
        os.environ.setdefault(k, v)                        # plain `python -m ...` = one rank
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    E, topk = args.experts, args.topk
    if args.small:
        T, H, F = 1024, 512, 1024
    elif args.mid:
        T, H, F = 4096, 2048, 4096
    else:
        T, H, F = args.tokens, 4096, 14336
    G = E // P
    cap_rows = int(T * topk * P / E * 1.25)
    # the heap's allocator hands out power-of-two blocks: two receive buffers (forward, backward), two per-entry
    # return buffers, the runtime's own region and small tables
    p2 = lambda n: 1 << max(n - 1, 1).bit_length()
    heap = 2 * p2((G * cap_rows + 256) * H * 2) + 2 * p2(T * topk * H * 2) + (1 << 30)
    rt = shmem.init("device", device=local, heap_bytes=heap, timeout_ms=20000)
    dev = rt.device
    torch.manual_seed(7)                                   # same weights on every rank, sliced per rank
    wr = torch.randn(E, H, device=dev).to(torch.bfloat16)
    w1 = (torch.randn(E, F, H, device=dev) * 0.02).to(torch.bfloat16)[rank * G:(rank + 1) * G].contiguous()
    w3 = (torch.randn(E, F, H, device=dev) * 0.02).to(torch.bfloat16)[rank * G:(rank + 1) * G].contiguous()
    w2 = (torch.randn(E, H, F, device=dev) * 0.02).to(torch.bfloat16)[rank * G:(rank + 1) * G].contiguous()
    torch.manual_seed(100 + rank)
    x = torch.randn(T, H, device=dev).to(torch.bfloat16)
    dout = torch.randn(T, H, device=dev).to(torch.bfloat16)

    layer = MoELayer(rt, H, F, E, topk, T, capacity_factor=1.25, training=True, timeout_ms=20000)
    layer.wr.copy_(wr)
    layer.w2.copy_(w2)
    for g in range(G):
        layer.w13[g].copy_(interleave_gate_up(w1[g], w3[g]))
    layer.sync_transposes()
    rt.set_blocking(False)                                 # stream-ordered like the NCCL baseline

    res = {"world": P, "tokens_per_rank": T, "hidden": H, "ffn": F, "experts": E, "topk": topk, "capacity_rows": layer.cap}
    y = layer.forward(x).clone()
    dx = layer.backward(dout).clone()
    torch.cuda.synchronize()
    layer.check()

    ok = True
    if not args.no_baseline:
        base = NcclMoE(wr, w1.clone(), w3.clone(), w2.clone(), topk, router_grad=True)   # same work as ours: router backward included
        xb = x.clone().requires_grad_(True)
        yb = base(xb)
        yb.backward(dout)
        torch.cuda.synchronize()
        sy, sdx = yb.detach().float().abs().max().item(), xb.grad.float().abs().max().item()
        ey = (y.float() - yb.detach().float()).abs().max().item()
        edx = (dx.float() - xb.grad.float()).abs().max().item()
        ew2 = (layer.dw2.float() - base.w2.grad.float()).abs().max().item() / (base.w2.grad.float().abs().max().item() + 1e-9)
        ok = ey <= 5e-2 * sy + 2e-2 and edx <= 8e-2 * sdx + 2e-2 and ew2 <= 8e-2
        res.update({"fwd_max_abs_diff": ey, "fwd_scale": sy, "dx_max_abs_diff": edx, "dx_scale": sdx, "dw2_rel_diff": ew2})

    def ours():
        layer.forward(x)
        layer.backward(dout)

    ms = timed(ours, args.iters, rt)
    layer.check()
    ms_f = timed(lambda: layer.forward(x), args.iters, rt)
    res.update({"ms_fwd_bwd": ms, "ms_fwd": ms_f})
    # useful FLOPs: 3 GEMM pairs forward (gate, up, down), twice that backward
    rows = float(layer.recv_count.sum().item())
    flops_fwd = 2.0 * rows * H * F * 3
    res["tflops_fwd_bwd_per_gpu"] = 3 * flops_fwd / (ms * 1e-3) / 1e12
    if not args.no_baseline:
        def theirs():
            xb2 = x.clone().requires_grad_(True)
            base.zero_grad(set_to_none=True)
            base(xb2).backward(dout)
        ms_b = timed(theirs, max(2, args.iters // 2), rt)
        with torch.no_grad():
            ms_bf = timed(lambda: base(x), max(2, args.iters // 2), rt)
        res.update({"ms_fwd_bwd_nccl_cublas": ms_b, "ms_fwd_nccl_cublas": ms_bf, "speedup_fwd_bwd": ms_b / ms, "speedup_fwd": ms_bf / ms_f})
    # ---- the all-to-all alone: dispatch (tokens -> experts) and combine (expert rows -> sources) against
    # NCCL all_to_all_single moving the same rows; device time of the exchange only, max over ranks ----
    import ctypes as C
    from roc_shmem_b200.ops.moe import SIG_FWD_COMBINE, SIG_FWD_DISPATCH, _stream
    lib = layer.lib
    n_entries = T * topk

    def a2a_ours(iters):
        td = tc = 0.0
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        for _ in range(iters):
            layer.route(x)                                   # new call parity, counts exchanged, arrival words armed
            par, s = layer.parity, _stream()
            rt.barrier_all()
            evs[0].record()
            lib.bshmem_moe_dispatch(C.byref(layer.state), C.byref(layer.plan), x.data_ptr(), 0, layer.topk_idx.data_ptr(),
                                    layer.pos.data_ptr(), n_entries, topk, H, layer.recv.data_ptr(), layer.meta.data_ptr(), par,
                                    SIG_FWD_DISPATCH, layer.ctas, s)
            lib.bshmem_moe_wait_arrivals(C.byref(layer.plan), par, SIG_FWD_DISPATCH, layer.expect_from.data_ptr(), 20000,
                                         layer.err_word, s)
            evs[1].record()
            rt.barrier_all()
            evs[2].record()
            lib.bshmem_moe_combine_send(C.byref(layer.state), C.byref(layer.plan), layer.recv.data_ptr(), layer.meta.data_ptr(), H,
                                        layer.ybuf.data_ptr(), par, SIG_FWD_COMBINE, layer.ctas, s)
            lib.bshmem_moe_wait_arrivals(C.byref(layer.plan), par, SIG_FWD_COMBINE, layer.send_to.data_ptr(), 20000,
                                         layer.err_word, s)
            evs[3].record()
            torch.cuda.synchronize()
            td += evs[0].elapsed_time(evs[1])
            tc += evs[2].elapsed_time(evs[3])
        t = torch.tensor([td / iters, tc / iters], device=dev)
        if P > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    a2a_ours(1)
    ms_disp, ms_comb = a2a_ours(args.iters)
    layer.check()
    link_bytes = n_entries * (P - 1) / P * H * 2
    res.update({"a2a_dispatch_ms": ms_disp, "a2a_combine_ms": ms_comb, "a2a_link_ms_at_770GBps": link_bytes / 770e9 * 1e3,
                "a2a_dispatch_frac_of_link": (link_bytes / 770e9 * 1e3) / ms_disp if P > 1 else None,
                "a2a_combine_frac_of_link": (link_bytes / 770e9 * 1e3) / ms_comb if P > 1 else None})
    if P > 1 and not args.no_baseline:
        # the same rows through NCCL: sorted by destination expert, split sizes from the routing
        idx = layer.topk_idx.view(T, topk).long()
        flat_e = idx.reshape(-1)
        order = torch.argsort(flat_e, stable=True)
        send = x[order // topk].contiguous()
        counts = torch.bincount(flat_e, minlength=E)
        recv_counts = torch.empty_like(counts)
        dist.all_to_all_single(recv_counts, counts)
        in_splits = counts.view(P, G).sum(1).tolist()
        out_splits = recv_counts.view(P, G).sum(1).tolist()
        recv_n = torch.empty((sum(out_splits), H), dtype=x.dtype, device=dev)
        back_n = torch.empty_like(send)
        ms_nd = timed(lambda: dist.all_to_all_single(recv_n, send, out_splits, in_splits), args.iters, rt)
        ms_nc = timed(lambda: dist.all_to_all_single(back_n, recv_n, in_splits, out_splits), args.iters, rt)
        res.update({"a2a_dispatch_ms_nccl": ms_nd, "a2a_combine_ms_nccl": ms_nc, "a2a_dispatch_speedup": ms_nd / ms_disp,
                    "a2a_combine_speedup": ms_nc / ms_comb})
    okt = torch.tensor([int(ok)], device=dev)
    dist.all_reduce(okt, op=dist.ReduceOp.MIN)
    res["all_ranks_ok"] = bool(okt.item())
    rt.synchronize()
    rt.set_blocking(True)
    if rank == 0:
        line = json.dumps(res)
        print(line, flush=True)
        if args.out:
            os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
            with open(args.out, "w") as f:
                f.write(line + "\n")
    shmem.finalize()
    dist.destroy_process_group()
    if not res["all_ranks_ok"]:
        raise SystemExit(1)


if __name__ == "__main__":
    main()
