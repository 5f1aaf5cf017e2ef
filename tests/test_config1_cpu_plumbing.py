"""2-PE host-centric plumbing on CPU threads + a shared-memory heap: 64 MiB
heap, int64 put of 1 Mi elements to the neighbour, barrier_all, int64 sum_to_all,
4 KiB fcollect and 1000 atomic fetch-adds on a uint64 counter; all bitwise."""
import torch

from roc_shmem_b200.cpu import run_threads

N = 1 << 20


def _pe_body(rt):
    me, n = rt.my_pe, rt.n_pes
    nbr = (me + 1) % n
    src = torch.arange(N, dtype=torch.int64) + me * (1 << 20)      # private (non-symmetric) source
    dst = rt.empty((N,), torch.int64)
    red_src = rt.empty((N,), torch.int64)
    red_dst = rt.empty((N,), torch.int64)
    fc_src = rt.empty((4096,), torch.uint8)
    fc_dst = rt.empty((4096 * n,), torch.uint8)
    counter = rt.zeros((1,), torch.int64)

    rt.put(dst, src, nbr)
    rt.barrier_all()
    left = (me - 1) % n
    assert torch.equal(dst, torch.arange(N, dtype=torch.int64) + left * (1 << 20))

    red_src.copy_(src)
    rt.reduce(red_dst, red_src, "sum")
    expect = sum(torch.arange(N, dtype=torch.int64) + p * (1 << 20) for p in range(n))
    assert torch.equal(red_dst, expect)

    fc_src.fill_(me + 1)
    rt.fcollect(fc_dst, fc_src)
    for p in range(n):
        assert bool((fc_dst[p * 4096:(p + 1) * 4096] == p + 1).all())

    seen = set()
    for _ in range(1000):
        seen.add(rt.atomic_fetch_add(counter, 1, 0))
    rt.barrier_all()
    total = rt.g(counter, 0)
    assert total == 1000 * n
    assert len(seen) == 1000          # every fetched value is distinct
    rt.barrier_all()
    return sorted(seen)


def test_config1_two_pes():
    res = run_threads(2, _pe_body, heap_bytes=64 << 20)
    # the two PEs' fetched tickets interleave to exactly 0..1999
    assert sorted(res[0] + res[1]) == list(range(2000))
