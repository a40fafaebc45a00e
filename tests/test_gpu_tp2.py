"""The engine at world_size 2 on the product library: two tensor-parallel ranks, one GPU each.

The reference pins this behaviour in pegaflow-server/tests/mock_vllm_rpc_e2e.rs:318-360 (a query
before every TP slot of a block has been saved is a miss, then a hit, then each rank loads its own
slots), pegaflow-core/src/instance.rs:757-825 (the topology seals once `world_size` GPUs have
registered; slot = layer * tp_size + tp_rank) and lease.rs:98,125-133 (a lease is consumed once per
rank).  An instance holds one context per device (a second registration of the same device is
refused, instance.rs:757-825), so the scenario needs two GPUs and skips on a single-GPU box."""
import numpy as np
import pytest

from oracle.engine_model import EngineError, OracleEngine
from tests import scenarios as sc
from tests.gpu_util import CudaMem

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pf():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device (there is no CPU fallback to test)")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs: one per tensor-parallel rank")
    import pegaflow_b200

    return pegaflow_b200


def _drive(eng, mems, err):
    """The same call sequence on either engine; returns what it observed."""
    seen = {}
    layers = {r: [sc.Layer(f"model.layers.{i}.attn", 16, 4096, segments=2, kv_stride=16 * 4096) for i in range(3)]
              for r in range(2)}
    sc.register(eng, mems[0], "tp", "ns", layers[0], device_id=0, tp_rank=0, tp_size=2, world_size=2)
    h = sc.make_block_hashes(3, 7)
    with pytest.raises(err, match="registration incomplete: 1/2 workers"):       # not sealed yet
        eng.batch_save("tp", 0, 0, 0, [(L.name, [1, 2, 3], h) for L in layers[0]])
    sc.register(eng, mems[1], "tp", "ns", layers[1], device_id=1, tp_rank=1, tp_size=2, world_size=2)
    with pytest.raises(err, match="already fully registered"):
        sc.register(eng, mems[1], "tp", "ns", [sc.Layer("extra", 4, 512)], device_id=2, tp_rank=1, tp_size=2, world_size=2)
    for r in range(2):
        for i, L in enumerate(layers[r]):
            mems[r].write(L.buf, sc.seeded_bytes(L.region_bytes, 100 + 10 * r + i))
    src = {0: [1, 2, 3], 1: [9, 4, 12]}          # the ranks hold the blocks at different ids
    dst = {0: [13, 14, 15], 1: [5, 6, 7]}
    eng.batch_save("tp", 0, 0, 0, [(L.name, src[0], h) for L in layers[0]])
    eng.flush_saves()
    seen["after_rank0"] = eng.query_prefix("tp", h)[1]                             # 3 missing: rank 1's slots are empty
    with pytest.raises(err, match="but save requested"):
        eng.batch_save("tp", 0, 0, 1, [(L.name, src[1], h) for L in layers[1]])    # device 1 is rank 1, not rank 0
    eng.batch_save("tp", 1, 0, 1, [(L.name, src[1], h) for L in layers[1]])
    eng.flush_saves()
    blocks, missing = eng.query_prefix("tp", h)
    seen["after_both"] = (len(blocks), missing)
    seen["slots"] = blocks[0].num_slots if hasattr(blocks[0], "num_slots") else len(blocks[0].slots)
    seen["images"] = [[bytes(x) for x in eng.block_slot_image("tp", hh, slot)] for hh in h for slot in range(6)]
    lease = eng.create_query_lease("tp", blocks)
    for r in range(2):
        for L in layers[r]:
            mems[r].zero(L.buf)
        eng.batch_load("tp", r, r, [[L.name for L in layers[r]]], [(lease, [dst[r]])])
        mems[r].sync()
    seen["lease_left"] = eng.release_query_lease(lease)                             # both ranks consumed it
    with pytest.raises(err, match="unknown or expired"):
        eng.batch_load("tp", 0, 0, [[L.name for L in layers[0]]], [(lease, [dst[0]])])
    seen["gpu"] = {(r, L.name): mems[r].read(L.buf) for r in range(2) for L in layers[r]}
    seen["expected"] = {(r, L.name): sc.expected_after_roundtrip(L, sc.seeded_bytes(L.region_bytes, 100 + 10 * r + i),
                                                                 src[r], dst[r])
                        for r in range(2) for i, L in enumerate(layers[r])}
    return seen


def test_tp2_seals_when_both_ranks_saved(pf):
    eng = pf.PegaEngine(32 << 20, min_dma_bytes=64 << 10)
    try:
        got = _drive(eng, {0: CudaMem(0), 1: CudaMem(1)}, pf.PegaFlowError)
        m = eng.metrics()
    finally:
        eng.close()
    want = _drive(OracleEngine(32 << 20), {0: sc.NumpyMem(), 1: sc.NumpyMem()}, EngineError)
    assert got["after_rank0"] == want["after_rank0"] == 3
    assert got["after_both"] == want["after_both"] == (3, 0)
    assert got["slots"] == want["slots"] == 6                  # 3 layers x tp_size 2
    assert got["images"] == want["images"], "a stored slot differs from the oracle (slot = layer * 2 + tp_rank)"
    assert got["lease_left"] is False and want["lease_left"] is False
    for key, expected in want["expected"].items():
        assert np.array_equal(want["gpu"][key], expected)
        assert np.array_equal(got["gpu"][key], expected), f"rank {key[0]} layer {key[1]} differs after the load"
    assert m["load_failures"] == 0 and m["load_tasks"] == 2 and m["save_batches"] == 2
