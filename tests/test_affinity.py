"""CPU placement helper: cpulist parsing and a no-op when the topology is unknown."""
from roc_shmem_b200.utils import affinity


def test_cpulist_parsing_and_missing_topology(tmp_path):
    assert affinity._parse_cpulist("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    assert affinity._parse_cpulist("") == set()
    assert affinity.local_cpus(0, sysfs=str(tmp_path)) is None        # no such device directory (or no GPU): unknown
