"""Fused TP kernels: single-PE degenerate case in-process, real multi-PE case as a
child torchrun job on 2 GPUs (skipped when only one GPU is visible)."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_fused_tp_single_pe():
    import roc_shmem_b200 as shmem
    from roc_shmem_b200.ops.fused_tp import AllGatherGemm, GemmReduceScatter
    rt = shmem.init("device", rank=0, world_size=1, heap_bytes=256 << 20)
    try:
        M, N, K = 512, 768, 320
        x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
        rs = GemmReduceScatter(rt, M, N, K)
        for _ in range(3):                       # several calls: parity buffers + monotonic signals
            rs(x, w)
        torch.cuda.synchronize()
        rs.check()
        ref = (x.float() @ w.float().t())
        assert (rs.out.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-3
        ag = AllGatherGemm(rt, M, N, K)
        ag.x_shard.copy_(x)
        for _ in range(2):
            ag(w)
        torch.cuda.synchronize()
        ag.check()
        assert (ag.out.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-3
        rs.close()
        ag.close()
    finally:
        shmem.finalize()


@pytest.mark.multigpu
def test_fused_tp_two_pes_against_nccl():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", B200SHMEM_NVLS="off", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29533", "-m", "roc_shmem_b200.bench.tp_bench", "--small", "--iters", "3"]
    p = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=280)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    line = [ln for ln in p.stdout.splitlines() if ln.startswith("{")][-1]
    res = json.loads(line)
    assert res["all_ranks_ok"] and res["ag_gather_exact"]
