"""Multi-GPU tests: child torchrun jobs on 2 GPUs (skipped when fewer are visible).
NVLS is switched off in NCCL and in the runtime for every job that may lose a rank."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _torchrun(nproc, args, port, timeout=280, nvls="off", extra_env=None):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT, B200SHMEM_NVLS=nvls)
    env.update(extra_env or {})
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


@pytest.mark.parametrize("nproc", [2, 4, 8])
def test_collectives_byte_exact(nproc):
    """fcollect / alltoall / broadcast / int32 reduce-scatter / allreduce, 1 KiB .. 64 MiB, three times back to back."""
    _need(nproc)
    p = _torchrun(nproc, ["tests/mp/coll_exact_worker.py"], 29620 + nproc, timeout=400)
    assert p.returncode == 0, p.stdout[-4000:] + p.stderr[-4000:]
    assert p.stdout.count("COLL_EXACT_OK") == nproc


def test_collectives_byte_exact_with_multicast():
    """The same checks with the NVLink multicast object bound: multimem.red barrier, multimem.st fcollect,
    in-switch allreduce.  No rank leaves in this job."""
    _need(2)
    p = _torchrun(2, ["tests/mp/coll_exact_worker.py"], 29631, timeout=400, nvls="auto",
                  extra_env={"COLL_EXACT_MAX_BYTES": str(32 << 20)})
    assert p.returncode == 0, p.stdout[-4000:] + p.stderr[-4000:]
    assert p.stdout.count("COLL_EXACT_OK") == 2


@pytest.mark.parametrize("backend", ["device", "proxy"])
def test_device_api_matrix_default_and_team_context(backend):
    """One kernel body, {default ctx, team ctx} x {NVLink, reverse-offload ring}: p/g, atomics, scoped RMA,
    put_signal, ordering and the work-group collectives of the context's team."""
    _need(2)
    p = _torchrun(2, ["tests/mp/api_matrix_worker.py"], 29640 + (1 if backend == "proxy" else 0), timeout=300,
                  extra_env={"API_MATRIX_BACKEND": backend})
    assert p.returncode == 0, p.stdout[-4000:] + p.stderr[-4000:]
    assert p.stdout.count("API_MATRIX_OK") == 2


@pytest.mark.parametrize("nproc", [2, 4])
def test_functional_driver_all_types(nproc):
    """Every type of the functional test driver between real PEs (sizes to 64 KiB, 4 work-groups of 128 threads)."""
    _need(nproc)
    p = _torchrun(nproc, ["-m", "roc_shmem_b200.bench.functional", "--all", "-w", "4", "-z", "128", "--loop", "20", "--skip", "4",
                          "--loop-large", "6"], 29650 + nproc, timeout=400)
    assert p.returncode == 0, p.stdout[-4000:] + p.stderr[-4000:]
    assert '"failed": []' in p.stdout
