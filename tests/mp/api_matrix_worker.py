"""The device API matrix over {default context, team context} on the transport named by API_MATRIX_BACKEND
("device" = NVLink loads/stores, "proxy" = reverse-offload ring), one rank per GPU under torchrun.
Prints "API_MATRIX_OK <rank>" on success."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import roc_shmem_b200 as shmem  # noqa: E402


def main() -> None:
    local = int(os.environ.get("LOCAL_RANK", 0))
    backend = os.environ.get("API_MATRIX_BACKEND", "device")
    torch.cuda.set_device(local)
    rt = shmem.init(backend, device=local, heap_bytes=256 << 20, timeout_ms=10000, proxy_slots=256)
    me, n = rt.my_pe, rt.n_pes
    use_proxy = backend == "proxy"
    bufs = rt.api_matrix_buffers(4096)
    # world context, PE numbers are world numbers
    rt.barrier_all()
    checks = rt.api_matrix(bufs, team=None, peer=(me + 1) % n, proxy=use_proxy)
    assert len(checks) == 25 and all(c == 1 for c in checks), f"[pe {me}] world ctx {backend}: {checks} {rt.error_record()}"
    rt.barrier_all()
    # a team with its own slot over all PEs in reverse... (start 0, stride 1, size n) and, with 4+ PEs, the even PEs
    team = rt.team_split_strided(None, 0, 1, n)
    checks = rt.api_matrix(bufs, team=team, peer=(team.my_pe + 1) % team.n_pes, proxy=use_proxy)
    assert len(checks) == 25 and all(c == 1 for c in checks), f"[pe {me}] team ctx {backend}: {checks} {rt.error_record()}"
    rt.barrier_all()
    team.destroy()
    if n >= 4:
        even = rt.team_split_strided(None, 0, 2, n // 2)
        if even.valid:
            checks = rt.api_matrix(bufs, team=even, peer=(even.my_pe + 1) % even.n_pes, proxy=use_proxy)
            assert len(checks) == 25 and all(c == 1 for c in checks), f"[pe {me}] even-team ctx {backend}: {checks}"
        rt.barrier_all()
        if even.valid:
            even.destroy()
    if use_proxy:
        rt.proxy.stop()
    shmem.finalize()
    print(f"API_MATRIX_OK {me}", flush=True)


if __name__ == "__main__":
    main()
