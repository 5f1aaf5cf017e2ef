"""Two-rank check of the model blocks (run under torchrun): the tensor-parallel Llama MLP (forward and
backward, all-gather→GEMM and GEMM→reduce-scatter fused kernels) and the expert-parallel MoE block against
fp32 PyTorch references of the unsharded math.  Prints "MODELS_OK <rank>"."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import roc_shmem_b200 as shmem  # noqa: E402
from roc_shmem_b200.models.llama import LlamaMLP, reference_mlp  # noqa: E402
from roc_shmem_b200.ops.moe import interleave_gate_up  # noqa: E402


def main() -> None:
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rt = shmem.init("device", device=local, heap_bytes=1 << 30, timeout_ms=8000)
    me, P = rt.my_pe, rt.n_pes
    dev = rt.device
    tol = lambda r: 3e-2 * r.abs().max().item() + 3e-2

    # ---- Llama MLP, TP = P, sequence-parallel activations ----
    M, H, F = 512 * P, 512, 512 * P
    Fp = F // P
    torch.manual_seed(11)                                     # same full tensors on every rank
    wg = (torch.randn(F, H, device=dev) * 0.05).to(torch.bfloat16)
    wu = (torch.randn(F, H, device=dev) * 0.05).to(torch.bfloat16)
    wd = (torch.randn(H, F, device=dev) * 0.05).to(torch.bfloat16)
    x = torch.randn(M, H, device=dev).to(torch.bfloat16)
    dy = torch.randn(M, H, device=dev).to(torch.bfloat16)
    block = LlamaMLP(rt, H, F, M)
    sl = slice(me * Fp, (me + 1) * Fp)
    block.load(wg[sl], wu[sl], wd[:, sl].contiguous())
    rows = slice(me * (M // P), (me + 1) * (M // P))
    for _ in range(2):                                        # twice: staging parity, monotonic signals
        y = block.forward(x[rows].contiguous()).clone()
        dx = block.backward(dy[rows].contiguous()).clone()
    torch.cuda.synchronize()
    block.check()
    xr, wgr, wur, wdr = (t.float().requires_grad_(True) for t in (x, wg, wu, wd))
    ref = reference_mlp(xr, wgr, wur, wdr)
    ref.backward(dy.float())
    assert (y.float() - ref.detach()[rows]).abs().max().item() <= tol(ref), "mlp forward"
    assert (dx.float() - xr.grad[rows]).abs().max().item() <= tol(xr.grad), "mlp dx"
    assert (block.dw2.float() - wdr.grad[:, sl]).abs().max().item() <= tol(wdr.grad), "mlp dw2"
    ref13 = interleave_gate_up(wgr.grad[sl], wur.grad[sl])
    assert (block.dw13.float() - ref13).abs().max().item() <= tol(ref13), "mlp dw13"
    rt.barrier_all()

    # ---- MoE block, EP = P ----
    from roc_shmem_b200.baseline.moe import moe_reference_single
    from roc_shmem_b200.models.mixtral import MixtralMoEBlock
    T, H2, F2, E, topk = 512, 256, 512, 8, 2
    G = E // P
    torch.manual_seed(12)
    wr = torch.randn(E, H2, device=dev).to(torch.bfloat16)
    w1 = (torch.randn(E, F2, H2, device=dev) * 0.05).to(torch.bfloat16)
    w3 = (torch.randn(E, F2, H2, device=dev) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(E, H2, F2, device=dev) * 0.05).to(torch.bfloat16)
    xs = [torch.randn(T, H2, device=dev).to(torch.bfloat16) for _ in range(P)]       # every rank's tokens
    dys = [torch.randn(T, H2, device=dev).to(torch.bfloat16) for _ in range(P)]
    moe = MixtralMoEBlock(rt, hidden=H2, ffn=F2, n_experts=E, topk=topk, max_tokens=T, capacity_factor=2.0)
    es = slice(me * G, (me + 1) * G)
    moe.load(wr, w1[es], w3[es], w2[es])
    for _ in range(2):
        y2 = moe.forward(xs[me]).clone()
        dx2 = moe.backward(dys[me]).clone()
    torch.cuda.synchronize()
    moe.check()
    xall = torch.cat(xs).float().requires_grad_(True)
    w2r = w2.float().requires_grad_(True)
    wrr = wr.float().requires_grad_(True)
    ref2, idx, _ = moe_reference_single(xall, wrr, w1.float(), w3.float(), w2r, topk, router_grad=True)
    ref2.backward(torch.cat(dys).float())
    mine = slice(me * T, (me + 1) * T)
    same = (moe.topk_idx.view(T, topk).long() == idx[mine]).all(-1)
    assert same.float().mean() > 0.99, "routing"
    assert (y2.float() - ref2.detach()[mine])[same].abs().max().item() <= tol(ref2), "moe forward"
    assert (dx2.float() - xall.grad[mine])[same].abs().max().item() <= 5e-2 * xall.grad.abs().max().item() + 3e-2, "moe dx"
    # expert weight gradients sum over all ranks' tokens; tokens whose routing flipped on a near-tie perturb them slightly
    assert (moe.dw2.float() - w2r.grad[es]).abs().max().item() <= 8e-2 * w2r.grad.abs().max().item() + 5e-2, "moe dw2"
    # router weights: every rank holds the gradient of its own tokens; the sum over ranks is the full gradient
    dwr_all = moe.dwr.float().clone()
    dist.all_reduce(dwr_all)
    assert (dwr_all - wrr.grad).abs().max().item() <= 8e-2 * wrr.grad.abs().max().item() + 5e-2, "moe dwr"
    rt.barrier_all()
    print(f"MODELS_OK {me}", flush=True)
    shmem.finalize()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
