"""tcgen05 bf16 GEMM against a plain fp32 PyTorch reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b):
    return a.float() @ b.float().t()


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (256, 256, 512), (512, 768, 1024), (384, 320, 200), (1000, 520, 136),
                                   (2048, 2048, 2048)])
def test_gemm_bf16_matches_fp32_reference(M, N, K):
    from roc_shmem_b200.ops.gemm import gemm_bf16, gemm_error_site
    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    out = gemm_bf16(a, b)
    torch.cuda.synchronize()
    assert gemm_error_site() == 0
    ref = _ref(a, b)
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 2e-2 * scale + 1e-2, f"max abs err {err} vs scale {scale}"
    # bf16 rounding of the fp32 result is the only expected difference
    assert torch.allclose(out.float(), ref.to(torch.bfloat16).float(), rtol=2e-2, atol=2e-2 * scale)


def test_gemm_bf16_identity_pattern():
    """A = I picks out rows of B: exposes any tile / swizzle / descriptor mix-up exactly."""
    from roc_shmem_b200.ops.gemm import gemm_bf16
    M = N = K = 512
    a = torch.eye(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.arange(N * K, device="cuda", dtype=torch.float32).reshape(N, K).remainder(251).to(torch.bfloat16)
    out = gemm_bf16(a, b)
    torch.cuda.synchronize()
    assert torch.equal(out, b.t().contiguous())
