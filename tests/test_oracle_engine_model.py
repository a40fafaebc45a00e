"""The oracle engine model replays the reference's integration scenarios on CPU memory
(pegaflow-core/tests/engine_basic.rs, prefix_semantics.rs, save_validation.rs)."""
import numpy as np
import pytest

from oracle.engine_model import EngineError, OracleEngine
from tests import scenarios as sc


def _engine(**kw):
    return OracleEngine(16 << 20, **kw)


def test_save_query_load_roundtrip():
    eng, mem = _engine(), sc.NumpyMem()
    L = sc.Layer("layer_0", 4, 1024)
    fill = sc.fill_pattern(4, 1024)
    out = sc.roundtrip(eng, mem, "test-roundtrip", "test-ns", [L], range(4), range(4), sc.make_block_hashes(4, 0),
                       fills=[fill])
    assert np.array_equal(out["layer_0"], fill)


def test_page_first_multi_layer_roundtrip_uneven_offsets():
    eng, mem = _engine(), sc.NumpyMem()
    layers = [sc.Layer("layer_a", 4, 512), sc.Layer("layer_b", 4, 1024), sc.Layer("layer_c", 4, 1536)]
    fills = [sc.fill_pattern(4, 512), sc.fill_pattern(4, 1024, 0x40), sc.fill_pattern(4, 1536, 0x80)]
    hashes = sc.make_block_hashes(4, 0xAB)
    out = sc.roundtrip(eng, mem, "test-page-first", "test-ns", layers, range(4), range(4), hashes, fills=fills,
                       page_first=True)
    for L, f in zip(layers, fills):
        assert np.array_equal(out[L.name], f)
    # the stored page of block 2 is layer_a | layer_b | layer_c at offsets 0, 512, 1536
    img = eng.block_slot_image("test-page-first", hashes[2], 0)
    assert len(img) == 1 and len(img[0]) == 3072
    assert img[0][:512] == bytes([3]) * 512 and img[0][512:1536] == bytes([3 + 0x40]) * 1024
    assert img[0][1536:] == bytes([3 + 0x80]) * 1536


def test_page_first_rejects_partial_layer_save():
    eng, mem = _engine(), sc.NumpyMem()
    layers = [sc.Layer(n, 4, 512) for n in ("layer_a", "layer_b", "layer_c")]
    sc.register(eng, mem, "pf-partial", "ns", layers, page_first=True)
    with pytest.raises(EngineError, match="must cover all"):
        eng.batch_save("pf-partial", 0, 0, 0, [("layer_a", [0, 1, 2, 3], sc.make_block_hashes(4, 0xCD))])


def test_hybrid_groups_load_to_distinct_block_ids(kats):
    eng, mem = _engine(), sc.NumpyMem()
    layers = [sc.Layer("full_attention", 4, 1024), sc.Layer("gdn", 4, 1024)]
    sc.register(eng, mem, "hyb", "ns", layers, use_groups=True)
    mem.write(layers[0].buf, sc.fill_pattern(4, 1024))
    mem.write(layers[1].buf, sc.fill_pattern(4, 1024, 0x40))
    hashes = sc.make_block_hashes(2, 0xAC)
    eng.batch_save("hyb", 0, 0, 0, [("full_attention", [0, 1], hashes), ("gdn", [2, 3], hashes)])
    for L in layers:
        mem.zero(L.buf)
    blocks, missing = eng.query_prefix("hyb", hashes)
    assert missing == 0
    lease = eng.create_query_lease("hyb", blocks)
    eng.batch_load("hyb", 0, 0, [["full_attention"], [], ["gdn"]],
                   [(lease, [[2, 3], [None, None], [None, 0]])])
    full = np.zeros(4096, dtype=np.uint8)
    full[2048:3072] = 1
    full[3072:4096] = 2
    gdn = np.zeros(4096, dtype=np.uint8)
    gdn[0:1024] = kats["engine_roundtrips"]["hybrid_expected"]["gdn"]["0"]
    assert np.array_equal(mem.read(layers[0].buf), full)
    assert np.array_equal(mem.read(layers[1].buf), gdn)


@pytest.mark.parametrize("seg,kv_stride,nblocks", [(512, 4096, 4), (4096, 16384, 2)])
def test_split_storage_roundtrip(seg, kv_stride, nblocks):
    eng, mem = _engine(), sc.NumpyMem()
    L = sc.Layer("layer_0", nblocks, seg, segments=2, kv_stride=kv_stride)
    fill = sc.seeded_bytes(L.region_bytes, 7)
    ids = list(range(nblocks))
    out = sc.roundtrip(eng, mem, "split", "ns", [L], ids, ids[::-1], sc.make_block_hashes(nblocks, 1), fills=[fill])
    assert np.array_equal(out["layer_0"], sc.expected_after_roundtrip(L, fill, ids, ids[::-1]))


def test_multi_layer_partial_save_is_not_a_hit_and_dedup():
    eng, mem = _engine(), sc.NumpyMem()
    layers = [sc.Layer("layer_0", 4, 1024), sc.Layer("layer_1", 4, 1024)]
    sc.register(eng, mem, "ml", "ns", layers)
    hashes = sc.make_block_hashes(4, 55)
    eng.batch_save("ml", 0, 0, 0, [("layer_0", [0, 1, 2, 3], hashes)])
    assert len(eng.query_prefix("ml", hashes)[0]) == 0
    eng.batch_save("ml", 0, 0, 0, [("layer_1", [0, 1, 2, 3], hashes)])
    assert len(eng.query_prefix("ml", hashes)[0]) == 4
    eng.batch_save("ml", 0, 0, 0, [("layer_0", [0, 1, 2, 3], hashes)])  # dedup: no new slots
    assert len(eng.query_prefix("ml", hashes)[0]) == 4


def test_prefix_semantics_gap_breaks_prefix():
    eng, mem = _engine(), sc.NumpyMem()
    layers = [sc.Layer("layer_0", 3, 1024)]      # kept: registered memory must outlive its use
    sc.register(eng, mem, "gap", "ns", layers)
    allh = sc.make_block_hashes(4, 20)
    eng.batch_save("gap", 0, 0, 0, [("layer_0", [0, 1, 2], [allh[0], allh[2], allh[3]])])
    blocks, missing = eng.query_prefix("gap", allh)
    assert (len(blocks), missing) == (1, 3)


def test_validation_errors():
    eng, mem = _engine(), sc.NumpyMem()
    with pytest.raises(EngineError, match="instance nope not found"):
        eng.batch_save("nope", 0, 0, 0, [])
    L = sc.Layer("layer_0", 4, 1024)
    sc.register(eng, mem, "v", "ns", [L], world_size=2, tp_size=2)
    with pytest.raises(EngineError, match="registration incomplete: 1/2"):
        eng.batch_save("v", 0, 0, 0, [("layer_0", [0], [b"h"])])
    L2 = sc.Layer("layer_0", 4, 1024)
    sc.register(eng, mem, "v", "ns", [L2], world_size=2, tp_size=2, device_id=1, tp_rank=1)
    with pytest.raises(EngineError, match="already exists"):
        sc.register(eng, mem, "v", "ns", [L2], world_size=2, tp_size=2, device_id=1, tp_rank=1)
    with pytest.raises(EngineError, match="already fully registered"):
        sc.register(eng, mem, "v", "ns", [L2], world_size=2, tp_size=2, device_id=2, tp_rank=1)
    with pytest.raises(EngineError, match="topology mismatch"):
        sc.register(eng, mem, "v", "ns", [L2], world_size=1, tp_size=2, device_id=3, tp_rank=1)
    with pytest.raises(EngineError, match="block_id 4 out of range"):
        eng.batch_save("v", 0, 0, 0, [("layer_0", [4], [b"h"])])
    with pytest.raises(EngineError, match="does not match block_hashes"):
        eng.batch_save("v", 0, 0, 0, [("layer_0", [1, 2], [b"h"])])
    with pytest.raises(EngineError, match="device 9 not found"):
        eng.batch_save("v", 0, 0, 9, [("layer_0", [1], [b"h"])])
    with pytest.raises(EngineError, match="but save requested"):
        eng.batch_save("v", 1, 0, 0, [("layer_0", [1], [b"h"])])


def test_layer_ids_follow_bytewise_name_order():
    eng, mem = _engine(), sc.NumpyMem()
    names = ["model.layers.10.attn", "model.layers.2.attn", "model.layers.1.attn"]
    layers = [sc.Layer(n, 2, 256) for n in names]
    sc.register(eng, mem, "ord", "ns", layers)
    topo = eng.instances["ord"].topology
    assert [topo.layer_id(n) for n in names] == [1, 2, 0]


def test_cleanup_memory_cache_counts_what_leaves_and_what_is_still_held():
    """storage/mod.rs:662-681: two resident blocks, one of them held elsewhere -> evicted 2, still referenced 1;
    a second clean-up finds nothing."""
    eng, mem = _engine(), sc.NumpyMem()
    L = sc.Layer("layer_0", 4, 1024)
    sc.register(eng, mem, "clean", "ns", [L])
    held, free = sc.make_block_hashes(1, 60), sc.make_block_hashes(1, 61)
    eng.batch_save("clean", 0, 0, 0, [("layer_0", [0], held)])
    eng.batch_save("clean", 0, 0, 0, [("layer_0", [1], free)])
    blocks, _ = eng.query_prefix("clean", held)
    lease = eng.create_query_lease("clean", blocks)
    assert eng.cleanup_memory_cache() == {"evicted_blocks": 2, "evicted_bytes": 2048, "still_referenced_blocks": 1}
    assert eng.query_prefix("clean", held) == ([], 1) and eng.query_prefix("clean", free) == ([], 1)
    assert eng.cleanup_memory_cache() == {"evicted_blocks": 0, "evicted_bytes": 0, "still_referenced_blocks": 0}
    assert eng.release_query_lease(lease) is True        # the lease outlives the cache entry


def test_stale_inflight_sweep_and_instance_listing():
    """lib.rs:938-948 (blocks whose missing slots never came are dropped after an age limit) and lib.rs:459-489
    (list, namespace, unregister all; leases go with the instances)."""
    import time

    eng, mem = _engine(), sc.NumpyMem()
    assert eng.list_instance_ids() == [] and eng.unregister_all_instances() == [] and eng.gc_stale_inflight(0.0) == 0
    layers = [sc.Layer("layer_0", 4, 1024), sc.Layer("layer_1", 4, 1024)]
    sc.register(eng, mem, "inst-b", "ns-1", layers)
    other = [sc.Layer("layer_0", 4, 1024)]
    sc.register(eng, mem, "inst-a", "ns-2", other)
    assert eng.list_instance_ids() == ["inst-a", "inst-b"] and eng.instance_namespace("inst-b") == "ns-1"
    with pytest.raises(EngineError) as e:
        eng.instance_namespace("nobody")
    assert e.value.kind == "InstanceMissing"
    hashes = sc.make_block_hashes(4, 77)
    eng.batch_save("inst-b", 0, 0, 0, [("layer_0", [0, 1, 2, 3], hashes)])     # layer_1 never comes
    assert eng.query_prefix("inst-b", hashes) == ([], 4)
    assert eng.gc_stale_inflight(300.0) == 0
    time.sleep(0.02)
    assert eng.gc_stale_inflight(0.01) == 4 and eng.gc_stale_inflight(0.0) == 0
    eng.batch_save("inst-b", 0, 0, 0, [("layer_0", [0, 1, 2, 3], hashes), ("layer_1", [0, 1, 2, 3], hashes)])
    blocks, missing = eng.query_prefix("inst-b", hashes)
    assert missing == 0
    lease = eng.create_query_lease("inst-b", blocks)
    with pytest.raises(EngineError):
        eng.gc_stale_inflight(-1.0)
    assert eng.unregister_all_instances() == ["inst-a", "inst-b"] and eng.list_instance_ids() == []
    assert eng.release_query_lease(lease) is False
