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
