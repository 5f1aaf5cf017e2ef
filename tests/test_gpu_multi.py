"""Multi-GPU tests: child torchrun jobs on 2 GPUs (skipped when fewer are visible).
NVLS is switched off in NCCL and in the runtime for every job that may lose a rank."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _torchrun(nproc, args, port, timeout=280):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT, B200SHMEM_NVLS="off")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
           "127.0.0.1", "--master-port", str(port)] + args
    return subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)


def _need(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def test_runtime_matrix_two_pes():
    _need(2)
    p = _torchrun(2, ["tests/mp/runtime_worker.py"], 29611)
    assert p.returncode == 0, p.stdout[-4000:] + p.stderr[-4000:]
    assert p.stdout.count("WORKER_OK") == 2


def test_rank_leaves_between_steps_peers_time_out():
    _need(2)
    p = _torchrun(2, ["tests/mp/failure_worker.py"], 29612)
    assert p.returncode == 0, p.stdout[-4000:] + p.stderr[-4000:]
    assert "SURVIVOR_SAW_TIMEOUT" in p.stdout


def test_model_blocks_two_pes():
    _need(2)
    p = _torchrun(2, ["tests/mp/models_worker.py"], 29613)
    assert p.returncode == 0, p.stdout[-4000:] + p.stderr[-4000:]
    assert p.stdout.count("MODELS_OK") == 2
