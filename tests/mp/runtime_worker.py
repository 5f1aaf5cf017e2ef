"""Multi-process functional matrix of the NVLink runtime (run under torchrun, one rank per GPU).

Follows the reference's functional test matrix (clients/functional_tests/tester.hpp:34-87):
put/get(+nbi) with closed-form verification, p/g, the atomic families, ping-pong, barrier /
sync, broadcast, reduction, fcollect, alltoall (value (src << 16) + dst identifies each block),
shmem_ptr, team-context RMA, team reduction/broadcast, and the extensions (put_signal,
reduce_scatter).  Prints "WORKER_OK <rank>" on success.
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import roc_shmem_b200 as shmem  # noqa: E402


def main() -> None:
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    rt = shmem.init("device", device=local, heap_bytes=512 << 20, timeout_ms=5000)
    me, n = rt.my_pe, rt.n_pes
    dev = rt.device
    nxt, prv = (me + 1) % n, (me - 1) % n
    assert rt.heap_mode in ("vmm", "ipc")

    # ---- put / get, blocking and nbi, host-initiated ----
    N = 1 << 18
    buf = rt.empty((N,), torch.int64)
    buf.fill_(-1)
    rt.barrier_all()
    src = torch.arange(N, device=dev, dtype=torch.int64) + me * (1 << 20)
    rt.put(buf, src, nxt)
    rt.barrier_all()
    assert torch.equal(buf, torch.arange(N, device=dev, dtype=torch.int64) + prv * (1 << 20)), "put"
    got = torch.empty_like(src)
    rt.get(got, buf, nxt, nbi=True)
    rt.quiet()
    assert torch.equal(got, torch.arange(N, device=dev, dtype=torch.int64) + me * (1 << 20)), "get_nbi"
    rt.barrier_all()

    # ---- device-initiated put / get at every scope ----
    big = rt.empty((4 << 20,), torch.uint8)
    pattern = (torch.arange(4 << 20, device=dev) * (me + 3) % 251).to(torch.uint8)
    for scope in ("thread", "warp", "block"):
        big.zero_()
        rt.barrier_all()
        rt.rma_kernel(big, pattern, nxt, put=True, scope=scope, ctas=8, threads=256)
        rt.barrier_all()
        expect = (torch.arange(4 << 20, device=dev) * (prv + 3) % 251).to(torch.uint8)
        assert torch.equal(big, expect), f"device put {scope}"
        out = torch.zeros_like(pattern)
        rt.rma_kernel(big, out, nxt, put=False, scope=scope, ctas=8, threads=256)
        rt.quiet()
        assert torch.equal(out, pattern), f"device get {scope}"      # nxt holds what I put there
        rt.barrier_all()
    local_out = torch.zeros(64 * 128 * 8, device=dev, dtype=torch.uint8)
    rt.swarm_get(local_out, big, 8, nxt, 64, 128)                     # every thread its own 8-byte get
    assert torch.equal(local_out, pattern[: local_out.numel()]), "swarm get"
    rt.barrier_all()

    # ---- typed device API inside one kernel: p/g, all 15 atomics, ptr, test ----
    checks = rt.api_selftest(nxt)
    assert len(checks) >= 17 and all(c == 1 for c in checks), f"api selftest {checks}"

    # ---- host atomics on a remote PE (closed-form totals) ----
    ctr = rt.zeros((2,), torch.int64)
    for _ in range(50):
        rt.atomic_fetch_add(ctr, 2, 0)
        rt.atomic_inc(ctr[1:], 0)
    rt.barrier_all()
    if me == 0:
        assert ctr.tolist() == [100 * n, 50 * n], ctr.tolist()
    rt.barrier_all()

    # ---- put_signal + wait_until hand-off around the ring ----
    data = rt.zeros((1024,), torch.float32)
    sig = rt.zeros((1,), torch.int64)
    payload = torch.full((1024,), float(me + 1), device=dev)
    rt.put_signal(data, payload, sig, 1, nxt)
    rt.wait_until(sig, "eq", 1)
    assert bool((data == float(prv + 1)).all()), "put_signal payload"
    rt.barrier_all()

    # ---- ping-pong latency kernel (pairs 0/1) and work-group collectives from a user kernel ----
    flag = rt.zeros((1,), torch.int64)
    if me < 2 and n >= 2:
        lat = rt.bench_pingpong(flag, 1 - me, 50, me == 0)
        assert 0.1 < lat < 200.0, lat
    rt.barrier_all()
    a = rt.empty((4096,), torch.float32)
    b = rt.zeros((4096,), torch.float32)
    a.fill_(1.0)
    rt.barrier_all()
    assert rt.wg_collectives(b, a) == 0
    assert bool((b == float(n)).all()), "wg_to_all: float sum of ones == n_pes"
    rt.barrier_all()

    # ---- collectives through the host API ----
    v = rt.empty((100_003,), torch.float32)
    r = rt.empty((100_003,), torch.float32)
    v.copy_(torch.full((100_003,), float(me + 1), device=dev))
    rt.reduce(r, v, "sum")
    assert bool((r == n * (n + 1) / 2).all()), "to_all sum"
    rt.reduce(v, v, "max")                                            # in place
    assert bool((v == float(n)).all()), "to_all max in place"
    bsrc = rt.empty((5000,), torch.int32)
    bdst = rt.empty((5000,), torch.int32)
    bsrc.fill_(me + 10)
    bdst.fill_(-7)
    rt.broadcast(bdst, bsrc, n - 1)
    assert bool((bdst == (-7 if me == n - 1 else n - 1 + 10)).all()), "broadcast (root's dest untouched)"
    blk = 3000
    asrc = rt.empty((blk * n,), torch.int32)
    adst = rt.empty((blk * n,), torch.int32)
    for j in range(n):
        asrc[j * blk:(j + 1) * blk] = (me << 16) + j
    rt.alltoall(adst, asrc)
    for j in range(n):
        assert bool((adst[j * blk:(j + 1) * blk] == (j << 16) + me).all()), "alltoall"
    fsrc = rt.empty((blk,), torch.int32)
    fdst = rt.empty((blk * n,), torch.int32)
    fsrc.fill_(me + 1)
    rt.fcollect(fdst, fsrc)
    for j in range(n):
        assert bool((fdst[j * blk:(j + 1) * blk] == j + 1).all()), "fcollect"
    rs_src = rt.empty((1000 * n,), torch.float32)
    rs_dst = rt.empty((1000,), torch.float32)
    rs_src.copy_(torch.arange(1000 * n, device=dev, dtype=torch.float32) + me)
    rt.reduce_scatter(rs_dst, rs_src, "sum")
    expect = n * (torch.arange(1000, device=dev, dtype=torch.float32) + me * 1000) + n * (n - 1) / 2
    assert torch.allclose(rs_dst, expect), "reduce_scatter"

    # ---- teams: even PEs, team-relative context RMA, team reduce ----
    if n >= 2:
        team = rt.team_split_strided(None, 0, 2, (n + 1) // 2)
        if me % 2 == 0:
            assert team.valid and team.my_pe == me // 2 and team.n_pes == (n + 1) // 2
            assert team.translate_pe(team.my_pe, rt.team_world) == me
            tv = rt.empty((512,), torch.float32, collective=False)
            tr = rt.empty((512,), torch.float32, collective=False)
        else:
            assert not team.valid
            tv = rt.empty((512,), torch.float32, collective=False)
            tr = rt.empty((512,), torch.float32, collective=False)
        tv.fill_(float(me))
        tr.zero_()
        rt.barrier_all()
        if team.valid:
            rt.reduce(tr, tv, "sum", team=team)
            assert bool((tr == float(sum(range(0, n, 2)))).all()), "team reduce"
            with rt.ctx_create(shmem.CTX_WG_PRIVATE, team) as ctx:
                nb = (team.my_pe + 1) % team.n_pes            # team-relative neighbour
                ctx.put(tr, tv, nb)
                ctx.quiet()
            team.sync()
            left = team.translate_pe((team.my_pe - 1) % team.n_pes, rt.team_world)
            assert bool((tr == float(left)).all()), "team ctx put"
            team.destroy()
        rt.barrier_all()

    # ---- bounded wait: a flag nobody sets comes back as a timeout, context stays usable ----
    from roc_shmem_b200.utils.timeouts import temporary_timeout
    never = rt.zeros((1,), torch.int64)
    try:
        with temporary_timeout(rt, 100):
            rt.wait_until(never, "eq", 1)
        raise AssertionError("wait_until on an unset flag must time out")
    except shmem.ShmemTimeout:
        rt.error_record()
    rt.barrier_all()
    st = rt.device_stats()
    assert st["barrier"] > 0
    print(f"WORKER_OK {me}", flush=True)
    shmem.finalize()


if __name__ == "__main__":
    main()
