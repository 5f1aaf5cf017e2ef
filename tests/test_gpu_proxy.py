"""Reverse-offload mode on the GPU: device kernels enqueue descriptors, the CPU thread executes
them; a paused service thread shows up on the device as a bounded-wait timeout."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_device_commands_through_the_ring_and_host_fault_injection():
    import roc_shmem_b200 as shmem
    rt = shmem.init("proxy", rank=0, world_size=1, heap_bytes=128 << 20, timeout_ms=5000, proxy_slots=64)
    try:
        px = rt.proxy
        checks = px.device_selftest(0, threads=96)               # 3 warps: warp-aggregated tickets
        assert len(checks) == 12 and all(c == 1 for c in checks), (checks, px.counters(), rt.error_record())
        c = px.counters()
        assert c["processed"] >= 96 + 10 and c["amo"] >= 96 and c["errors"] == 0
        x = rt.zeros((8,), torch.int64)
        with pytest.raises(shmem.ShmemError):                     # host threads use the host API, not a GPU ring
            px.put(x, torch.arange(8, device="cuda"), 0)
        # a paused service thread: the device-side wait gives up with TIMEOUT, the context stays usable
        px.set_timeout_ms(100)
        px.pause(True)
        assert px.device_expect_timeout(x, 0) == 3               # BSHMEM_ERR_TIMEOUT
        rec = rt.error_record()
        assert rec["code"] == 3 and rec["where"] == 5            # BSHMEM_WHERE_PROXY_DONE
        before = px.counters()["processed"]
        px.pause(False)
        px.set_timeout_ms(5000)
        import time
        t0 = time.time()
        while px.counters()["processed"] == before and time.time() - t0 < 5:
            time.sleep(0.01)
        torch.cuda.synchronize()
        assert int(x[0]) == 1                                    # the stalled fetch-add ran once the thread resumed
        y = torch.ones(4, device="cuda")
        assert float((y * 2).sum()) == 8.0
    finally:
        rt.proxy.stop()
        shmem.finalize()


@pytest.mark.parametrize("backend", ["device", "proxy"])
def test_device_api_matrix_single_pe(backend):
    """The whole device API matrix on one PE (peer = self): direct transport and through the ring, world context and
    a team context (a team over the single PE has its own slot, so the team paths run)."""
    import roc_shmem_b200 as shmem
    rt = shmem.init(backend, rank=0, world_size=1, heap_bytes=256 << 20, timeout_ms=5000, proxy_slots=128)
    try:
        bufs = rt.api_matrix_buffers(2048)
        use_proxy = backend == "proxy"
        checks = rt.api_matrix(bufs, peer=0, proxy=use_proxy)
        assert len(checks) == 25 and all(c == 1 for c in checks), (checks, rt.error_record())
        team = rt.team_split_strided(None, 0, 1, 1)
        checks = rt.api_matrix(bufs, team=team, peer=0, proxy=use_proxy)
        assert len(checks) == 25 and all(c == 1 for c in checks), (checks, rt.error_record())
        team.destroy()
    finally:
        if backend == "proxy":
            rt.proxy.stop()
        shmem.finalize()
