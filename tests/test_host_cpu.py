"""Host-side helpers of the host-buffer front end that need no GPU."""
import os

from inference_b200.host import bind_to_device_numa_node, rank_rows


def test_rank_rows_cover_a_panel_in_rank_order():
    assert [rank_rows(2048, 4, r) for r in range(4)] == [(0, 512), (512, 1024), (1024, 1536), (1536, 2048)]


def test_numa_binding_follows_the_device_node(tmp_path):
    allowed = sorted(os.sched_getaffinity(0))
    dev = tmp_path / "0000:1b:00.0"
    dev.mkdir()
    (dev / "numa_node").write_text("1\n")
    # the device's CPUs: the first allowed CPU and some that this process may not use at all
    (dev / "local_cpulist").write_text(f"{allowed[0]},100000-100003\n")
    try:
        got = bind_to_device_numa_node("00000000:1B:00.0\n", sysfs_root=str(tmp_path))
        assert got == {"node": 1, "cpus": 1}
        assert os.sched_getaffinity(0) == {allowed[0]}
    finally:
        os.sched_setaffinity(0, allowed)


def test_numa_binding_changes_nothing_without_topology(tmp_path):
    before = os.sched_getaffinity(0)
    assert bind_to_device_numa_node("0000:1b:00.0", sysfs_root=str(tmp_path)) is None      # no such device
    dev = tmp_path / "0000:1b:00.0"
    dev.mkdir()
    (dev / "numa_node").write_text("-1\n")
    (dev / "local_cpulist").write_text("0-3\n")
    assert bind_to_device_numa_node("0000:1b:00.0", sysfs_root=str(tmp_path)) is None      # no NUMA information
    assert bind_to_device_numa_node("garbage", sysfs_root=str(tmp_path)) is None
    assert os.sched_getaffinity(0) == before
