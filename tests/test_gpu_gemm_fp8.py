"""Block-scaled fp8 tcgen05 GEMM and its quantisers against fp32 PyTorch references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref_quant(x: torch.Tensor, block_rows: int):
    """fp32 reference of the quantiser: per (block_rows x 128) block absmax / 448, e4m3 round-to-nearest."""
    R, K = x.shape
    xb = x.float().view(R // block_rows, block_rows, K // 128, 128)
    amax = xb.abs().amax(dim=(1, 3), keepdim=True)
    scale = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    q = (xb / scale).to(torch.float8_e4m3fn)
    return q.view(R, K), scale.view(R // block_rows, K // 128)


def test_quantisers_match_reference():
    from roc_shmem_b200.ops.gemm_fp8 import quantize_act, quantize_weight
    torch.manual_seed(0)
    x = (torch.randn(384, 512, device="cuda") * 3).to(torch.bfloat16)
    x[5, 128:256] = 0                                        # an all-zero block gets scale 1
    qa = quantize_act(x)
    rq, rs = _ref_quant(x, 1)
    torch.cuda.synchronize()
    assert torch.allclose(qa.scales.t(), rs, rtol=1e-6)
    # division vs multiplication by the reciprocal may flip a rounding tie here and there
    assert (qa.q.view(torch.float8_e4m3fn).float() == rq.float()).float().mean() > 0.999
    assert (qa.dequantize() - x.float()).abs().max().item() <= x.float().abs().max().item() * 0.07
    w = torch.randn(256, 384, device="cuda").to(torch.bfloat16)
    qw = quantize_weight(w)
    rq, rs = _ref_quant(w, 128)
    torch.cuda.synchronize()
    assert torch.allclose(qw.scales.t(), rs, rtol=1e-6)
    assert (qw.q.view(torch.float8_e4m3fn).float() == rq.float()).float().mean() > 0.999
    assert (qw.dequantize() - w.float()).abs().max().item() <= w.float().abs().max().item() * 0.07


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (256, 512, 384), (1024, 1792, 2048), (19 * 128, 3 * 256, 640)])
def test_gemm_fp8_blockscale(M, N, K):
    from roc_shmem_b200.ops.gemm_fp8 import fp8_error_site, gemm_fp8, quantize_act, quantize_weight
    torch.manual_seed(M + N + K)
    # row- and block-dependent magnitudes so that wrong scale indexing shows
    x = (torch.randn(M, K, device="cuda") * (1 + torch.arange(M, device="cuda").view(M, 1) % 7)).to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * (0.02 * (1 + torch.arange(N, device="cuda").view(N, 1) // 128 % 5))).to(torch.bfloat16)
    qa, qw = quantize_act(x), quantize_weight(w)
    out = torch.full((M, N), 7.0, dtype=torch.bfloat16, device="cuda")
    for _ in range(2):
        gemm_fp8(qa, qw, out)
    torch.cuda.synchronize()
    assert fp8_error_site() == 0
    ref = qa.dequantize() @ qw.dequantize().t()              # same quantised operands, fp32 math
    err = (out.float() - ref).abs().max().item()
    assert err <= 1e-2 * ref.abs().max().item() + 1e-3, err
    # and the quantised product stays close to the bf16 one
    full = x.float() @ w.float().t()
    assert (out.float() - full).abs().max().item() <= 0.06 * full.abs().max().item()


def test_all_gather_gemm_fp8_single_pe_equals_plain_kernel():
    """With one PE the fused kernel has nothing to pull: same tiles, same math, bit-identical output; run twice
    (call-parity counters)."""
    import roc_shmem_b200 as shmem
    from roc_shmem_b200.ops.gemm_fp8 import AllGatherGemmFp8, gemm_fp8, quantize_act, quantize_weight
    rt = shmem.init("device", rank=0, world_size=1, heap_bytes=256 << 20, timeout_ms=5000)
    try:
        torch.manual_seed(5)
        M, N, K = 512, 768, 640
        x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        qw = quantize_weight((torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16))
        op = AllGatherGemmFp8(rt, M, N, K)
        for _ in range(2):
            op.set_input(x)
            op(qw)
        torch.cuda.synchronize()
        op.check()
        qa = quantize_act(x)
        assert torch.equal(op.xq, qa.q) and torch.equal(op.sa, qa.scales)
        assert torch.equal(op.out, gemm_fp8(qa, qw))
        op.close()
    finally:
        shmem.finalize()


def test_gemm_reduce_scatter_fp8_single_pe_equals_plain_kernel():
    """One PE: the partial tiles go through the staging slot and the in-kernel reduction of a single partial;
    the result must equal the plain fp8 GEMM bit for bit, on both call parities."""
    import roc_shmem_b200 as shmem
    from roc_shmem_b200.ops.gemm_fp8 import GemmReduceScatterFp8, gemm_fp8, quantize_act, quantize_weight
    rt = shmem.init("device", rank=0, world_size=1, heap_bytes=256 << 20, timeout_ms=5000)
    try:
        torch.manual_seed(6)
        M, N, K = 640, 512, 384
        qa = quantize_act(torch.randn(M, K, device="cuda").to(torch.bfloat16))
        qw = quantize_weight((torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16))
        op = GemmReduceScatterFp8(rt, M, N, K)
        ref = gemm_fp8(qa, qw)
        for _ in range(3):
            op.out.fill_(7.0)
            op(qa, qw)
            torch.cuda.synchronize()
            op.check()
            assert torch.equal(op.out, ref)
        op.close()
    finally:
        shmem.finalize()


def test_gemm_reduce_scatter_fp8_one_k_block_per_tile():
    """K = 128 is a single k-block, so a tile is finished as soon as it is started and the epilogue warps of a block
    run several tiles apart: the per-tile publish counters (four, indexed by tile ordinal) must not mix tiles.
    512 tiles of 128 x 256 on 148 blocks; checked against the plain kernel (bit for bit) and a float32 reference."""
    import roc_shmem_b200 as shmem
    from roc_shmem_b200.ops.gemm_fp8 import GemmReduceScatterFp8, gemm_fp8, quantize_act, quantize_weight
    rt = shmem.init("device", rank=0, world_size=1, heap_bytes=512 << 20, timeout_ms=5000)
    try:
        torch.manual_seed(16)
        M, N, K = 8192, 2048, 128
        x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
        qa, qw = quantize_act(x), quantize_weight(w)
        op = GemmReduceScatterFp8(rt, M, N, K)
        ref = gemm_fp8(qa, qw)
        full = x.float() @ w.float().t()
        for _ in range(3):
            op.out.fill_(7.0)
            op(qa, qw)
            torch.cuda.synchronize()
            op.check()
            assert torch.equal(op.out, ref)
        assert (op.out.float() - full).abs().max().item() <= 0.06 * full.abs().max().item()
        op.close()
    finally:
        shmem.finalize()
