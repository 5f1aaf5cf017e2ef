"""The functional test driver's table of test types (bench/functional.py) against the kernel source: every type number the
kernels switch on has exactly one table row, the numbers are the reference's (clients/functional_tests/tester.hpp:34-87;
15 is retired there), and look-ups by number and by name agree."""
import re
from pathlib import Path

from roc_shmem_b200.bench.functional import BY_ID, SPECS, Tester, lookup

SRC = Path(__file__).resolve().parents[1] / "roc_shmem_b200" / "csrc" / "cuda" / "functional_tester.cu"


def test_table_is_complete_and_ordered():
    ids = [s.id for s in SPECS]
    assert ids == sorted(ids) and len(set(ids)) == len(ids) == 52 and 15 not in ids
    assert lookup("2").name == "put" and lookup("wg_put_nbi").id == 31 and lookup("52").name == "put_signal"
    assert len({s.name for s in SPECS}) == len(SPECS)


def test_table_matches_kernel_enum():
    text = SRC.read_text()
    enum = text[text.index("enum FtType {"):text.index("FT_COUNT")]
    numbers = sorted(int(n) for n in re.findall(r"FT_[A-Z_0-9]+ = (\d+)", enum))
    assert numbers == sorted(BY_ID)
    assert "FT_COUNT = 53" in text


def test_size_sweep_doubles_up_to_the_limit():
    t = Tester.__new__(Tester)            # sizes() needs no runtime
    t.max_size, t.n, t.span, t.wgs, t.wg_size = 1 << 20, 2, 4 << 20, 4, 64
    assert t.sizes(BY_ID[2], 1, 1 << 20) == [1 << k for k in range(21)]
    assert t.sizes(BY_ID[26], 1, 64) == [1, 2, 4, 8]
    assert t.sizes(BY_ID[6], 1, 1 << 20) == [8]
    assert t.sizes(BY_ID[5], 1, 4096)[0] == 4 and t.sizes(BY_ID[4], 1, 1 << 20)[-1] == 4096
