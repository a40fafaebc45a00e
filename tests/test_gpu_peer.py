"""GPU -> GPU block copy for same-box prefix hits.  With one GPU the source and destination
instances live on the same device (same kernel, same addressing); with two or more GPUs the source
is a peer device reached over NVLink."""
import numpy as np
import pytest

from tests import scenarios as sc
from tests.gpu_util import CudaMem

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device (there is no CPU fallback to test)")
    import pegaflow_b200 as pf

    return pf, torch


def _peer_roundtrip(pf, torch, src_dev, dst_dev):
    eng = pf.PegaEngine(32 << 20)
    try:
        # Qwen3-32B TP4 shard shape: 2 KV heads per rank, HND inside a block is still one 8 KiB segment
        n_layers, num_blocks, seg = 3, 128, 16 * 2 * 128 * 2
        rng = np.random.default_rng(17)
        mems = {src_dev: CudaMem(src_dev), dst_dev: CudaMem(dst_dev)}
        a = [sc.Layer(f"model.layers.{i}.attn", num_blocks, seg, segments=2, kv_stride=num_blocks * seg) for i in range(n_layers)]
        b = [sc.Layer(f"model.layers.{i}.attn", num_blocks, seg, segments=2, kv_stride=num_blocks * seg) for i in range(n_layers)]
        sc.register(eng, mems[src_dev], "inst-a", "ns", a, device_id=src_dev)
        sc.register(eng, mems[dst_dev], "inst-b", "ns", b, device_id=dst_dev)
        fills = [sc.seeded_bytes(L.region_bytes, 30 + i) for i, L in enumerate(a)]
        for L, f in zip(a, fills):
            mems[src_dev].write(L.buf, f)
        src_ids = (rng.permutation(num_blocks - 1)[:40] + 1).tolist()
        dst_ids = (rng.permutation(num_blocks - 1)[:40] + 1).tolist()
        eng.peer_load("inst-a", src_dev, "inst-b", dst_dev, src_ids, dst_ids)
        for L, f in zip(b, fills):
            want = sc.expected_after_roundtrip(L, f, src_ids, dst_ids)
            assert np.array_equal(mems[dst_dev].read(L.buf), want)
        with pytest.raises(pf.PegaflowInvalidArgument, match="out of range"):
            eng.peer_load("inst-a", src_dev, "inst-b", dst_dev, [num_blocks], [1])
        with pytest.raises(pf.PegaflowInvalidArgument, match="one destination per source"):
            eng.peer_load("inst-a", src_dev, "inst-b", dst_dev, [1, 2], [1])
        m = eng.metrics()["transfer"]
        assert m["bytes_peer"] == n_layers * 40 * 2 * seg and m["device_status"] == 0
    finally:
        eng.close()


def test_peer_load_between_instances_on_one_device(env):
    pf, torch = env
    _peer_roundtrip(pf, torch, 0, 0)


def test_peer_load_over_nvlink(env):
    pf, torch = env
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _peer_roundtrip(pf, torch, 0, 1)
    _peer_roundtrip(pf, torch, 1, 0)


def test_prefix_hit_between_instances_in_two_processes_over_nvlink(env):
    """The way instances really meet: each is its own process.  This process is instance A (GPU 0); it
    exports its layers' regions like the reference ships KV handles (python/pegaflow/ipc_wrapper.py:101-163);
    a child process is instance B on GPU 1, opens them and pulls blocks across NVLink."""
    import ctypes as C
    import json
    import os
    import pickle
    import subprocess
    import sys
    import tempfile

    pf, torch = env
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from pegaflow_b200 import _native as N

    nb, seg, n_layers, seed = 256, 16 * 2 * 128 * 2, 5, 600
    dev = torch.device("cuda", 0)
    layers = [torch.from_numpy(np.random.default_rng(seed + l).integers(0, 256, size=(2, nb, seg), dtype=np.uint8)).to(dev)
              for l in range(n_layers)]
    torch.cuda.synchronize()
    regions = []
    for t in layers:
        r = N.IpcRegion()
        N.check(N.lib.pf_ipc_export(t.data_ptr(), t.numel(), C.byref(r)))
        regions.append(bytes(r))
    rng = np.random.default_rng(9)
    job = dict(regions=regions, dst_device=1, num_blocks=nb, seg=seg, seed=seed,
               src_ids=(rng.permutation(nb - 1)[:100] + 1).tolist(), dst_ids=(rng.permutation(nb - 1)[:100] + 1).tolist())
    with tempfile.NamedTemporaryFile(suffix=".pkl", delete=False) as f:
        pickle.dump(job, f)
        path = f.name
    try:
        proc = subprocess.run([sys.executable, os.path.join(os.path.dirname(os.path.abspath(__file__)), "peer_child.py"), path],
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=300)
    finally:
        os.unlink(path)
    lines = [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]
    assert proc.returncode == 0 and lines, proc.stderr[-3000:]
    out = json.loads(lines[-1])
    assert out["bit_exact"] and out["device_status"] == 0
    assert out["bytes_peer"] == n_layers * 100 * 2 * seg and out["kernel_launches"] == 1
    del layers


def test_peer_copy_rejects_ids_outside_a_stated_cache_size(env):
    pf, torch = env
    mem = CudaMem(0)
    a, b = mem.alloc(8 * 4096), mem.alloc(8 * 4096)
    be = pf.TransferBackend(0)
    try:
        with pytest.raises(pf.PegaflowInvalidArgument, match="block_id 8 out of range"):
            be.peer_copy((a.data_ptr(), 4096, 0, 4096, 1, 8), [1, 8], (b.data_ptr(), 4096, 0, 4096, 1, 8), [2, 3], 0)
        with pytest.raises(pf.PegaflowInvalidArgument, match="block_id 9 out of range"):
            be.peer_copy((a.data_ptr(), 4096, 0, 4096, 1), [1, 2], (b.data_ptr(), 4096, 0, 4096, 1, 8), [2, 9], 0)
        assert be.stats()["kernel_launches"] == 0
    finally:
        be.close()


def test_backend_peer_copy_unaligned_geometry(env):
    """Block sizes that are not a multiple of 16 fall back to the ld/st kernel."""
    pf, torch = env
    mem = CudaMem(0)
    n, bb = 20, 1001
    src, dst = mem.alloc(n * bb), mem.alloc(n * bb)
    data = sc.seeded_bytes(n * bb, 3)
    mem.write(src, data)
    be = pf.TransferBackend(0)
    sids, dids = [3, 7, 19, 0], [1, 2, 3, 4]
    be.peer_copy((src.data_ptr(), bb, 0, bb, 1), sids, (dst.data_ptr(), bb, 0, bb, 1), dids, 0)
    mem.sync()
    want = np.zeros(n * bb, dtype=np.uint8)
    for s_, d_ in zip(sids, dids):
        want[d_ * bb:(d_ + 1) * bb] = data[s_ * bb:(s_ + 1) * bb]
    assert np.array_equal(mem.read(dst), want)
    be.close()


def test_backend_peer_copy_layers_mixed_geometry(env):
    """Layers with different block sizes, one of them not a multiple of 16 bytes, in one call: the
    aligned ones share launches of the warp kernel, the odd one takes the byte path; more (layer,
    range) units than one launch holds."""
    pf, torch = env
    mem = CudaMem(0)
    rng = np.random.default_rng(23)
    nb, n = 96, 50
    shapes = [(8192, 2)] * 60 + [(1001, 1), (4096, 2), (2064, 1)] + [(8192, 2)] * 3   # 60*2 units > 96 per launch
    sids = (rng.permutation(nb)[:n]).astype(np.uint32)
    dids = (rng.permutation(nb)[:n]).astype(np.uint32)
    srcs, dsts, fills, s_lay, d_lay = [], [], [], [], []
    for i, (bb, ranges) in enumerate(shapes):
        region = ranges * nb * bb
        a, b = mem.alloc(region), mem.alloc(region)
        f = sc.seeded_bytes(region, 900 + i)
        mem.write(a, f)
        mem.zero(b)
        srcs.append(a), dsts.append(b), fills.append(f)
        s_lay.append((a.data_ptr(), bb, nb * bb, bb, ranges))
        d_lay.append((b.data_ptr(), bb, nb * bb, bb, ranges))
    be = pf.TransferBackend(0)
    before = be.stats()["kernel_launches"]
    be.peer_copy_layers(s_lay, sids, d_lay, dids, 0)
    mem.sync()
    for (bb, ranges), f, b in zip(shapes, fills, dsts):
        want = np.zeros(ranges * nb * bb, dtype=np.uint8)
        for r in range(ranges):
            for s_, d_ in zip(sids.tolist(), dids.tolist()):
                want[(r * nb + d_) * bb:(r * nb + d_ + 1) * bb] = f[(r * nb + s_) * bb:(r * nb + s_ + 1) * bb]
        assert np.array_equal(mem.read(b), want), f"block size {bb} x {ranges} ranges differs"
    st = be.stats()
    assert st["device_status"] == 0
    assert st["bytes_peer"] == sum(bb * ranges for bb, ranges in shapes) * n
    # 120 units of 8 KiB -> 2 launches, the byte-path layer 1, 4 KiB 1, 2064 B 1, the last three 8 KiB layers 1
    assert st["kernel_launches"] - before == 6
    be.close()
