"""Pinned-pool backing strategies on a GPU box (pegaflow-core/src/pinned_mem.rs:403-436:
test_allocate_cuda_host_alloc, test_allocate_regular, test_zero_size_fails, test_read_hugepage_size)
and per-node pools on a fake two-node sysfs tree.  Every strategy must hand out memory the copy
engine and the kernels can use at once, so each case ends in a save -> load round trip compared
with the oracle."""
import ctypes as C
import os

import numpy as np
import pytest

from oracle.engine_model import OracleEngine
from pegaflow_b200 import _native as N
from tests import scenarios as sc
from tests.gpu_util import CudaMem, host_view


def _free_huge_pages():
    try:
        for line in open("/proc/meminfo"):
            if line.startswith("HugePages_Free:"):
                return int(line.split()[1])
    except OSError:
        pass
    return 0


def test_zero_size_fails():
    """pinned_mem.rs:421-430; needs no GPU: the size is checked before any CUDA call."""
    for kw in ({}, {"use_mmap": 1}, {"use_hugepages": 1}):
        cfg = N.PoolConfig(kw.get("use_hugepages", 0), kw.get("use_mmap", 0), -1, 0, 1)
        h = C.c_void_p()
        assert N.lib.pf_pool_new(0, C.byref(cfg), C.byref(h)) == 5
        assert b"must be greater than zero" in N.lib.pf_last_error()


@pytest.fixture(scope="module")
def pf():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device (there is no CPU fallback to test)")
    import pegaflow_b200

    return pegaflow_b200


STRATEGIES = {"cuda_host_alloc": {}, "mmap_register": {"use_mmap": True}, "hugepages": {"use_hugepages": True},
              "mmap_transparent_huge": {"transparent_huge": True}}


@pytest.mark.gpu
@pytest.mark.parametrize("strategy", list(STRATEGIES))
def test_pool_strategy_allocates_usable_pinned_memory(pf, strategy):
    import torch

    if strategy == "hugepages" and _free_huge_pages() * N.lib.pf_huge_page_size() < (8 << 20):
        pytest.skip("no huge pages reserved on this box (HugePages_Free is 0); the box's setting is left alone")
    pool = pf.PinnedPool(8 << 20, **STRATEGIES[strategy])
    try:
        used, total, largest = pool.usage()
        assert total >= (8 << 20) - 512 and used == 0
        host, host_dev, handle = pool.alloc(4096)                  # test_allocate_cuda_host_alloc / _regular
        assert host and host_dev and pool.usage()[0] >= 4096
        pool.release(handle)
        # the memory works for both routes: DMA (copy engine) and zero-copy (kernel through host_dev)
        n, seg = 48, 16384
        host, host_dev, handle = pool.alloc(n * seg)
        mem = CudaMem(0)
        dev = mem.alloc(64 * seg)
        init = sc.seeded_bytes(64 * seg, 5)
        mem.write(dev, init)
        ids = np.random.default_rng(1).permutation(64)[:n]
        stream = torch.cuda.Stream()
        for route in (1, 2):
            host_view(host, n * seg)[:] = 0
            be = pf.TransferBackend(0, route=route, min_dma_bytes=64 << 10)
            x = [pf.LayerXfer(dev.data_ptr(), seg, 0, seg, 1, ids.tolist(), [[pf.HostRun(0, n, host, host_dev, seg)]])]
            be.save_layers(x, stream.cuda_stream)
            stream.synchronize()
            assert np.array_equal(host_view(host, n * seg).reshape(n, seg), init.reshape(64, seg)[ids])
            mem.zero(dev)
            be.load_layers(x, stream.cuda_stream)
            stream.synchronize()
            want = np.zeros_like(init).reshape(64, seg)
            want[ids] = init.reshape(64, seg)[ids]
            assert np.array_equal(mem.read(dev), want.reshape(-1))
            assert be.stats()["device_status"] == 0
            be.close()
        pool.release(handle)
    finally:
        pool.close()


@pytest.mark.gpu
def test_mmap_pool_pages_are_resident_after_pre_touch(pf):
    """pinned_mem.rs:343-376: every page of an mmap-backed pool has been touched (and so placed on a
    node) before it is registered; move_pages reports a node for each of them."""
    pool = pf.PinnedPool(4 << 20, use_mmap=True)
    try:
        host, _, handle = pool.alloc(4 << 20)
        page = os.sysconf("SC_PAGESIZE")
        addrs = (C.c_void_p * 8)(*[host + i * ((4 << 20) // 8) // page * page for i in range(8)])
        nodes = (C.c_int * 8)(*([-9] * 8))
        assert N.lib.pf_numa_query_pages(addrs, 8, nodes) == 0
        if os.path.isdir("/sys/devices/system/node/node0"):
            assert all(n >= 0 for n in nodes), list(nodes)
        pool.release(handle)
    finally:
        pool.close()


@pytest.mark.gpu
@pytest.mark.parametrize("backing", ["mmap", "hugepages"])
def test_engine_on_an_mmap_or_hugepage_pool_round_trips_like_the_oracle(pf, backing):
    if backing == "hugepages" and _free_huge_pages() * N.lib.pf_huge_page_size() < (16 << 20):
        pytest.skip("no huge pages reserved on this box (HugePages_Free is 0); the box's setting is left alone")
    kw = {"use_mmap_pool": True} if backing == "mmap" else {"use_hugepages": True}
    eng = pf.PegaEngine(16 << 20, min_dma_bytes=64 << 10, **kw)
    ora = OracleEngine(16 << 20)
    try:
        spec = [dict(name=f"l{i}", num_blocks=32, segment_bytes=4096, segments=2, kv_stride=32 * 4096) for i in range(3)]
        fills = [sc.seeded_bytes(2 * 32 * 4096, 40 + i) for i in range(3)]
        save_ids, load_ids, hashes = [3, 9, 17, 30, 1], [4, 5, 6, 7, 8], sc.make_block_hashes(5, 9)
        got = sc.roundtrip(eng, CudaMem(0), "i", "ns", [sc.Layer(**s) for s in spec], save_ids, load_ids, hashes, fills=fills)
        want = sc.roundtrip(ora, sc.NumpyMem(), "i", "ns", [sc.Layer(**s) for s in spec], save_ids, load_ids, hashes,
                            fills=fills)
        for name in want:
            assert np.array_equal(got[name], want[name])
        for h in hashes:
            for slot in range(3):
                assert [bytes(x) for x in eng.block_slot_image("i", h, slot)] == \
                       [bytes(x) for x in ora.block_slot_image("i", h, slot)]
    finally:
        eng.close()


@pytest.fixture
def two_node_sysfs(tmp_path):
    """A host with two NUMA nodes whose CPUs both exist on this machine; the GPU's PCI device sits on node 1."""
    import torch

    node = tmp_path / "devices" / "system" / "node"
    cpus = sorted(os.sched_getaffinity(0))
    half = max(1, len(cpus) // 2)
    for i, part in enumerate((cpus[:half], cpus[half:] or cpus[:half])):
        (node / f"node{i}").mkdir(parents=True)
        (node / f"node{i}" / "cpulist").write_text(",".join(map(str, part)) + "\n")
    (node / "online").write_text("0-1\n")
    p = torch.cuda.get_device_properties(0)
    bdf = "%04x:%02x:%02x.0" % (p.pci_domain_id, p.pci_bus_id, p.pci_device_id)   # cudaDeviceGetPCIBusId's form
    dev = tmp_path / "bus" / "pci" / "devices" / bdf
    dev.mkdir(parents=True)
    (dev / "numa_node").write_text("1\n")
    assert N.lib.pf_numa_set_sysfs_root(str(tmp_path).encode()) == 0
    yield tmp_path
    assert N.lib.pf_numa_set_sysfs_root(None) == 0


@pytest.mark.gpu
def test_per_node_pools_serve_the_gpus_own_node(pf, two_node_sysfs):
    """pinned_pool.rs:464-605 + lib.rs:144-166: with NUMA affinity on and more than one node, the pool is
    split over the nodes that have GPUs and a GPU's saves come out of its own node's share."""
    assert pf.numa_node_of_device(0) == 1 and N.lib.pf_numa_num_nodes() == 2
    eng = pf.PegaEngine(8 << 20, enable_numa_affinity=True, min_dma_bytes=64 << 10)
    try:
        fill = sc.seeded_bytes(16 * 8192, 3)
        L = sc.Layer("l0", 16, 8192)
        got = sc.roundtrip(eng, CudaMem(0), "n", "ns", [L], [1, 2, 3], [9, 8, 7], sc.make_block_hashes(3, 2), fills=[fill])
        assert np.array_equal(got["l0"], sc.expected_after_roundtrip(L, fill, [1, 2, 3], [9, 8, 7]))
        m = eng.metrics()
        assert m["pool_capacity_bytes"] <= 8 << 20 and m["pool_used_bytes"] >= 3 * 8192
    finally:
        eng.close()
