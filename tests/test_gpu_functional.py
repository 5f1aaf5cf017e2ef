"""The functional test driver (bench/functional.py + csrc/cuda/functional_tester.cu) on one GPU: every test type runs
its size sweep against the PE itself and verifies the moved bytes / closed-form atomic results.
Parity: the reference's driver script runs each type of its single test binary (clients/functional_tests/driver.sh:62-170)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tester():
    import roc_shmem_b200 as shmem
    from roc_shmem_b200.bench.functional import Tester
    rt = shmem.init("device", device=0, heap_bytes=256 << 20)
    t = Tester(rt, max_size=16384, wgs=3, wg_size=64, loop=12, skip=3, loop_large=5, large=4096)
    yield t
    t.close()
    shmem.finalize()


def _ids():
    from roc_shmem_b200.bench.functional import SPECS
    return [s.name for s in SPECS]


@pytest.mark.parametrize("name", _ids())
def test_every_type_single_pe(tester, name):
    from roc_shmem_b200.bench.functional import BY_NAME
    res = tester.run(BY_NAME[name], min_size=1, verbose=False)
    assert res["ok"], res
    assert all(r["kernel_ms"] >= 0 for r in res["rows"])
    if BY_NAME[name].family in ("rma", "mr", "amo", "pg", "coll"):
        assert all(r["latency_us"] > 0 for r in res["rows"]), res


def test_bad_arguments_are_rejected(tester):
    from roc_shmem_b200 import ShmemError
    t = tester
    with pytest.raises(ShmemError):
        t.rt.functional_run(15, size=8, wgs=1, wg_size=64, loops=1, skip=0, peer=0, sym_a=t.sym_a, sym_b=t.sym_b, local=t.local,
                            words=t.words, timers=t.timers, status=t.status)
    with pytest.raises(ShmemError):
        t.rt.functional_run(5, size=64, wgs=2, wg_size=64, loops=1, skip=0, peer=0, sym_a=t.sym_a, sym_b=t.sym_b, local=t.local,
                            words=t.words, timers=t.timers, status=t.status)
    assert torch.cuda.is_available()
