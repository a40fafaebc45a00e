"""NUMA helpers of the product library (csrc/numa.cpp) on a fake sysfs tree, through the C ABI.

The cases are the reference's own unit tests (pegaflow-common/src/numa.rs:505-604: cpulist range,
list, mixed, hyper-threading, empty, single; pinning an unknown node fails; GPU nodes are valid,
sorted and unique; the first id the driver's tool reports wins) plus the sysfs lookups this
library uses in place of that tool.  No GPU is needed."""
import ctypes as C
import os

import pytest

from pegaflow_b200 import _native as N


def _ints(fn, *args, capacity=256):
    out, n = (C.c_int * capacity)(), C.c_size_t()
    st = fn(*args, out, capacity, C.byref(n))
    return st, [out[i] for i in range(min(n.value, capacity))]


def parse(text):
    st, cpus = _ints(N.lib.pf_numa_parse_cpulist, text.encode())
    assert st == 0, N.lib.pf_last_error()
    return cpus


@pytest.fixture
def fake_sysfs(tmp_path):
    """Two nodes: node 0 = CPUs 0-1 (this process can run there), node 1 = CPUs 100000-100003 (it cannot),
    GPUs 0000:1b:00.0 on node 0, 0000:9c:00.0 on node 1, 0000:c8:00.0 unknown (-1, as a VM reports)."""
    node = tmp_path / "devices" / "system" / "node"
    (node / "node0").mkdir(parents=True)
    (node / "node1").mkdir()
    (node / "online").write_text("0-1\n")
    cpus = sorted(os.sched_getaffinity(0))[:2]
    (node / "node0" / "cpulist").write_text(",".join(map(str, cpus)) + "\n")
    (node / "node1" / "cpulist").write_text("100000-100003\n")
    pci = tmp_path / "bus" / "pci" / "devices"
    for bdf, n in (("0000:1b:00.0", 0), ("0000:9c:00.0", 1), ("0000:c8:00.0", -1)):
        (pci / bdf).mkdir(parents=True)
        (pci / bdf / "numa_node").write_text(f"{n}\n")
    assert N.lib.pf_numa_set_sysfs_root(str(tmp_path).encode()) == 0
    yield tmp_path, cpus
    assert N.lib.pf_numa_set_sysfs_root(None) == 0


def test_parse_cpulist_reference_cases():
    assert parse("0-3") == [0, 1, 2, 3]                       # numa.rs:518-522
    assert parse("0,4,8") == [0, 4, 8]                        # :524-528
    assert parse("0-2,8,16-17") == [0, 1, 2, 8, 16, 17]       # :530-534
    ht = parse("0-15,32-47")                                  # :536-544
    assert len(ht) == 32 and (ht[0], ht[15], ht[16], ht[31]) == (0, 15, 32, 47)
    assert parse("") == []                                    # :546-550
    assert parse("5") == [5]                                  # :552-556
    assert parse("3,1,1-2") == [1, 2, 3]                      # sorted, each once (numa.rs:164-165)


@pytest.mark.parametrize("text,why", [("0-1-2", "Invalid CPU range format: 0-1-2"), ("a", "Invalid CPU ID: a"),
                                      ("0,,1", "Invalid CPU ID: "), ("4-x", "Invalid CPU ID: x")])
def test_parse_cpulist_rejects_malformed_text_with_the_reference_messages(text, why):
    st, _ = _ints(N.lib.pf_numa_parse_cpulist, text.encode())
    assert st == 3
    assert N.lib.pf_last_error().decode() == "invalid argument: " + why


def test_parse_cpulist_reports_the_count_when_the_buffer_is_too_small():
    st, _ = _ints(N.lib.pf_numa_parse_cpulist, b"0-7", capacity=4)
    assert st == 3 and b"8 entries do not fit" in N.lib.pf_last_error()


def test_pin_unknown_node_fails():
    assert N.lib.pf_numa_pin_thread_to_node(-1) == 3          # numa.rs:511-516
    assert "unknown" in N.lib.pf_last_error().decode()


def test_gpu_numa_nodes_are_valid_sorted_unique():
    nodes = (C.c_int * 5)(3, 3, -1, 0, 5)                     # numa.rs:558-582
    out, n = (C.c_int * 5)(), C.c_size_t()
    assert N.lib.pf_numa_distinct_valid_nodes(nodes, 5, out, C.byref(n)) == 0
    assert [out[i] for i in range(n.value)] == [0, 3, 5]


def test_closest_cpu_numa_node_uses_first_reported_id():
    f = N.lib.pf_numa_parse_closest_cpu_node                   # numa.rs:584-594
    assert f(b"NUMA ID of closest CPU: 3\n") == 3
    assert f(b"NUMA IDs of closest CPU: 1,18-33\n") == 1
    assert f(b"") == -1 and f(b"no colon here") == -1 and f(b"NUMA ID of closest CPU: N/A\n") == -1


def test_topology_is_read_from_the_sysfs_tree(fake_sysfs):
    _, cpus = fake_sysfs
    assert N.lib.pf_numa_num_nodes() == 2
    assert _ints(N.lib.pf_numa_cpus_of_node, 0) == (0, cpus)
    assert _ints(N.lib.pf_numa_cpus_of_node, 1) == (0, [100000, 100001, 100002, 100003])
    assert _ints(N.lib.pf_numa_cpus_of_node, 7) == (0, [])
    assert N.lib.pf_numa_node_of_pci_device(b"0000:1b:00.0") == 0
    assert N.lib.pf_numa_node_of_pci_device(b"0000:9C:00.0") == 1      # CUDA reports bus ids in upper case
    assert N.lib.pf_numa_node_of_pci_device(b"0000:c8:00.0") == -1
    assert N.lib.pf_numa_node_of_pci_device(b"0000:ff:00.0") == -1


def test_pinning_restricts_the_thread_to_the_nodes_cpus(fake_sysfs):
    import threading

    _, cpus = fake_sysfs
    seen = {}

    def body():
        seen["rc"] = N.lib.pf_numa_pin_thread_to_node(0)
        seen["affinity"] = sorted(os.sched_getaffinity(0))       # pid 0 = the calling thread
        seen["rc_missing"] = N.lib.pf_numa_pin_thread_to_node(7)
        seen["why_missing"] = N.lib.pf_last_error().decode()
        seen["rc_offline"] = N.lib.pf_numa_pin_thread_to_node(1)  # CPUs this machine does not have
        seen["why_offline"] = N.lib.pf_last_error().decode()

    t = threading.Thread(target=body)
    t.start()
    t.join()
    assert seen["rc"] == 0 and seen["affinity"] == cpus
    assert seen["rc_missing"] == 3 and seen["why_missing"] == "invalid argument: No CPUs found for NUMA node 7"
    assert seen["rc_offline"] == 3 and "sched_setaffinity failed" in seen["why_offline"]


def test_sysfs_root_falls_back_to_the_real_tree():
    assert N.lib.pf_numa_set_sysfs_root(b"") == 0
    real = len([d for d in os.listdir("/sys/devices/system/node") if d.startswith("node") and d[4:].isdigit()]) \
        if os.path.isdir("/sys/devices/system/node") else 0
    assert N.lib.pf_numa_num_nodes() == real


def test_query_pages_reports_the_node_of_touched_memory():
    empty = (C.c_int * 1)()
    assert N.lib.pf_numa_query_pages(None, 0, empty) == 0       # numa.rs:596-600
    buf = (C.c_uint8 * 8192)()
    buf[0] = buf[4096] = 1                                      # numa.rs:602-616: touched memory has a node
    addrs = (C.c_void_p * 2)(C.addressof(buf), C.addressof(buf) + 4096)
    nodes = (C.c_int * 2)(-5, -5)
    assert N.lib.pf_numa_query_pages(addrs, 2, nodes) == 0
    assert all(n >= -1 for n in nodes)
    if os.path.isdir("/sys/devices/system/node/node0"):
        assert all(n >= 0 for n in nodes)


def test_pre_touch_worker_count_follows_the_reference_rule():
    cpus = len(os.sched_getaffinity(0))                          # pinned_mem.rs:378-391
    f = N.lib.pf_pool_pre_touch_threads
    assert f(4096) == 1 and f(1 << 30) == 1
    assert f((1 << 30) + 1) == min(2, cpus)
    assert f(5 << 30) == min(5, cpus)
    assert f(1 << 50) == cpus


def test_read_hugepage_size():
    assert N.lib.pf_huge_page_size() > 0                         # pinned_mem.rs:432-436
    assert N.lib.pf_huge_page_size() % 4096 == 0


def test_parse_cpulist_round_trips_any_set_of_cpus():
    """Property: whatever set of CPUs the kernel's list syntax spells - runs as ranges, singletons, in any order,
    overlapping - the parser gives back exactly that set, sorted."""
    from hypothesis import given, settings
    from hypothesis import strategies as st

    @settings(max_examples=200, deadline=None)
    @given(st.lists(st.tuples(st.integers(0, 240), st.integers(0, 12)), min_size=0, max_size=12), st.randoms())
    def check(runs, rnd):
        want, parts = set(), []
        for start, extra in runs:
            want.update(range(start, start + extra + 1))
            parts.append(str(start) if extra == 0 and rnd.random() < 0.7 else f"{start}-{start + extra}")
        rnd.shuffle(parts)
        assert parse(",".join(parts)) == sorted(want)

    check()
