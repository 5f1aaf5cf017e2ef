"""Model blocks and the PyTorch operator layer on one GPU against plain fp32 PyTorch with autograd."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    import roc_shmem_b200 as shmem
    r = shmem.init("device", rank=0, world_size=1, heap_bytes=1 << 30, timeout_ms=5000)
    yield r
    shmem.finalize()


def test_custom_op_linear_forward_backward():
    from roc_shmem_b200.ops.torch_ops import Linear
    torch.manual_seed(0)
    lin = Linear(512, 768, device="cuda")
    x = torch.randn(4, 64, 512, device="cuda").to(torch.bfloat16).requires_grad_(True)
    y = lin(x)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.detach().float().requires_grad_(True)
    wr = lin.weight.detach().float().requires_grad_(True)
    yr = xr @ wr.t()
    yr.backward(dy.float())
    assert y.shape == (4, 64, 768)
    assert (y.float() - yr).abs().max().item() <= 2e-2 * yr.abs().max().item() + 1e-2
    assert (x.grad.float() - xr.grad).abs().max().item() <= 2e-2 * xr.grad.abs().max().item() + 1e-2
    assert (lin.weight.grad.float() - wr.grad).abs().max().item() <= 2e-2 * wr.grad.abs().max().item() + 1e-2
    # odd shapes take the transposing fall-back of the weight gradient
    lin2 = Linear(136, 72, device="cuda")
    x2 = torch.randn(40, 136, device="cuda").to(torch.bfloat16).requires_grad_(True)
    lin2(x2).sum().backward()
    ref = torch.ones(40, 72, device="cuda").t() @ x2.detach().float()
    assert (lin2.weight.grad.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-2
    torch.library.opcheck(torch.ops.bshmem.linear, (x2.detach(), lin2.weight.detach()), test_utils=("test_schema", "test_faketensor"))


def test_custom_op_linear_fp8():
    torch.manual_seed(1)
    import roc_shmem_b200.ops.torch_ops  # noqa: F401  (registers the ops)
    x = torch.randn(256, 512, device="cuda").to(torch.bfloat16)
    w = (torch.randn(512, 512, device="cuda") * 0.05).to(torch.bfloat16)
    y = torch.ops.bshmem.linear_fp8(x, w)
    ref = x.float() @ w.float().t()
    assert (y.float() - ref).abs().max().item() <= 0.06 * ref.abs().max().item()


@pytest.mark.parametrize("via_autograd", [False, True])
def test_llama_mlp_single_pe(rt, via_autograd):
    from roc_shmem_b200.models.llama import LlamaMLP, LlamaMLPModule, reference_mlp
    from roc_shmem_b200.ops.moe import interleave_gate_up
    torch.manual_seed(2)
    M, H, F = 512, 512, 768
    wg = (torch.randn(F, H, device="cuda") * 0.05).to(torch.bfloat16)
    wu = (torch.randn(F, H, device="cuda") * 0.05).to(torch.bfloat16)
    wd = (torch.randn(H, F, device="cuda") * 0.05).to(torch.bfloat16)
    x = torch.randn(M, H, device="cuda").to(torch.bfloat16)
    dy = torch.randn(M, H, device="cuda").to(torch.bfloat16)
    if via_autograd:
        mod = LlamaMLPModule(rt, H, F, M)
        block = mod.block
        block.load(wg, wu, wd)
        xin = x.clone().requires_grad_(True)
        y = mod(xin)
        y.backward(dy)
        dx, dw13, dw2 = xin.grad, mod.w13.grad, mod.w2.grad
    else:
        block = LlamaMLP(rt, H, F, M)
        block.load(wg, wu, wd)
        y = block.forward(x).clone()
        dx = block.backward(dy)
        dw13, dw2 = block.dw13, block.dw2
    torch.cuda.synchronize()
    block.check()
    xr, wgr, wur, wdr = (t.float().requires_grad_(True) for t in (x, wg, wu, wd))
    ref = reference_mlp(xr, wgr, wur, wdr)
    ref.backward(dy.float())
    tol = lambda r: 3e-2 * r.abs().max().item() + 2e-2
    assert (y.float() - ref).abs().max().item() <= tol(ref)
    assert (dx.float() - xr.grad).abs().max().item() <= tol(xr.grad)
    assert (dw2.float() - wdr.grad).abs().max().item() <= tol(wdr.grad)
    ref13 = interleave_gate_up(wgr.grad, wur.grad)
    assert (dw13.float() - ref13).abs().max().item() <= tol(ref13)


def test_mixtral_block_autograd(rt):
    from roc_shmem_b200.baseline.moe import moe_reference_single
    from roc_shmem_b200.models.mixtral import MixtralMoEModule
    torch.manual_seed(3)
    T, H, F, E, topk = 512, 256, 512, 8, 2
    mod = MixtralMoEModule(rt, hidden=H, ffn=F, n_experts=E, topk=topk, max_tokens=T, capacity_factor=2.0)
    wr = torch.randn(E, H, device="cuda").to(torch.bfloat16)
    w1 = (torch.randn(E, F, H, device="cuda") * 0.05).to(torch.bfloat16)
    w3 = (torch.randn(E, F, H, device="cuda") * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(E, H, F, device="cuda") * 0.05).to(torch.bfloat16)
    mod.block.load(wr, w1, w3, w2)
    x = torch.randn(T, H, device="cuda").to(torch.bfloat16).requires_grad_(True)
    y = mod(x)
    dy = torch.randn_like(y)
    y.backward(dy)
    torch.cuda.synchronize()
    mod.block.check()
    xr = x.detach().float().requires_grad_(True)
    w2r = w2.float().requires_grad_(True)
    wrr = wr.float().requires_grad_(True)
    ref, idx, _ = moe_reference_single(xr, wrr, w1.float(), w3.float(), w2r, topk, router_grad=True)
    ref.backward(dy.float())
    same = (mod.block.topk_idx.view(T, topk).long() == idx).all(-1)
    assert same.float().mean() > 0.99
    assert (y.float() - ref.detach())[same].abs().max().item() <= 3e-2 * ref.abs().max().item() + 2e-2
    assert (x.grad.float() - xr.grad)[same].abs().max().item() <= 5e-2 * xr.grad.abs().max().item() + 2e-2
    assert (mod.w2.grad.float() - w2r.grad).abs().max().item() <= 5e-2 * w2r.grad.abs().max().item() + 5e-2
    # the router's weights get their gradient through the softmax over the chosen experts
    assert (mod.wr.grad.float() - wrr.grad).abs().max().item() <= 8e-2 * wrr.grad.abs().max().item() + 5e-2
