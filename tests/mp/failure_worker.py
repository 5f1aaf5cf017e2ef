"""Failure detection without a GPU fault: the last rank leaves between steps (none of its
kernels in flight); the survivors' next barrier runs into its short bound and comes back as
ShmemTimeout, their CUDA context stays usable.  Plain peer loads/stores only (no multimem)."""
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import roc_shmem_b200 as shmem  # noqa: E402


def main() -> None:
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    rt = shmem.init("device", device=local, heap_bytes=64 << 20, timeout_ms=5000, nvls="off")
    me, n = rt.my_pe, rt.n_pes
    x = rt.zeros((1024,), torch.float32)
    rt.barrier_all()                       # step 1: everybody is here
    torch.cuda.synchronize()
    if me == n - 1:
        # leave between steps: nothing of ours is in flight; tell the others on the host
        rt.bootstrap.store.set("left", str(me))
        torch.cuda.synchronize()
        print("LEAVER_EXITS", flush=True)
        os._exit(0)
    rt.bootstrap.store.get("left")         # the survivors learn of it on the host ...
    from roc_shmem_b200.utils.timeouts import temporary_timeout
    t0 = time.time()
    try:
        with temporary_timeout(rt, 300):   # ... and the next collective is bounded anyway
            rt.barrier_all()
        print("UNEXPECTED_BARRIER_SUCCESS", flush=True)
        os._exit(3)
    except shmem.ShmemTimeout:
        dt = time.time() - t0
        rec = rt.error_record()
        assert rec["where"] == 2 and rec["pe"] == n - 1, rec
        assert dt < 5.0, dt
    # the context is still good: local work and RMA to live peers keep working
    x.fill_(float(me))
    torch.cuda.synchronize()
    assert float(x.sum()) == 1024.0 * me
    print("SURVIVOR_SAW_TIMEOUT", flush=True)
    os._exit(0)                            # skip the collective finalize: a member is gone


if __name__ == "__main__":
    main()
