"""torch.ops.bshmem collectives (custom ops with fake + autograd registration) on the CPU backend."""
import torch

import roc_shmem_b200 as shmem
import roc_shmem_b200.ops.torch_ops as tops
from roc_shmem_b200.cpu import run_threads


def test_collective_custom_ops_forward_and_autograd():
    def body(rt):
        shmem.set_current(rt)
        me, n = rt.my_pe, rt.n_pes
        x = (torch.arange(6, dtype=torch.float32).view(6, 1) + 10 * me).repeat(1, 4).requires_grad_(True)
        y = torch.ops.bshmem.all_reduce(x, "sum")
        assert torch.equal(y, sum((torch.arange(6, dtype=torch.float32).view(6, 1) + 10 * p).repeat(1, 4) for p in range(n)))
        assert torch.equal(torch.ops.bshmem.all_reduce(x.detach(), "max"), x.detach() - 10 * me + 10 * (n - 1))
        g = torch.ops.bshmem.all_gather(x)
        assert g.shape == (6 * n, 4) and all(float(g.detach()[6 * p, 0]) == 10 * p for p in range(n))
        r = torch.ops.bshmem.reduce_scatter(g)                    # every PE holds the same g: slice me times n
        assert torch.equal(r, g[6 * me:6 * (me + 1)].detach() * n)
        a = torch.ops.bshmem.all_to_all((torch.arange(2 * n, dtype=torch.float32) + 100 * me).view(2 * n, 1))
        assert [float(a[2 * p, 0]) for p in range(n)] == [100.0 * p + 2 * me for p in range(n)]
        # autograd: d/dx sum(all_gather(x) * w) = reduce_scatter(w)
        w = torch.arange(6 * n * 4, dtype=torch.float32).view(6 * n, 4)
        (g * w).sum().backward()
        assert torch.equal(x.grad, n * w[6 * me:6 * (me + 1)])
        rt.barrier_all()
        tops.release_scratch()
        assert rt.heap_usage()["live_blocks"] == 0
    run_threads(3, body, heap_bytes=1 << 20, timeout_s=120)


def test_fake_implementations_give_shapes():
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        x = torch.empty(8, 16, dtype=torch.bfloat16)
        w = torch.empty(32, 16, dtype=torch.bfloat16)
        assert torch.ops.bshmem.linear(x, w).shape == (8, 32)
        assert torch.ops.bshmem.linear_wgrad(torch.empty(8, 32, dtype=torch.bfloat16), x).shape == (32, 16)
        assert torch.ops.bshmem.linear_fp8(x, w).shape == (8, 32)
        assert torch.ops.bshmem.all_reduce(x).shape == (8, 16)
