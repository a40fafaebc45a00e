"""Engine-level parity: the same call sequence is replayed on the CUDA engine (through the C ABI)
and on the CPU oracle model; GPU bytes after the load, every stored block's host image and the
error behaviour must agree.  Scenarios follow the reference's integration tests
(pegaflow-core/tests/engine_basic.rs, prefix_semantics.rs, save_validation.rs)."""
import numpy as np
import pytest

from oracle.engine_model import EngineError, OracleEngine
from tests import scenarios as sc
from tests.gpu_util import CudaMem, make_event

pytestmark = pytest.mark.gpu

ROUTES = {"auto": 0, "staged": 1, "zerocopy": 2}


@pytest.fixture(scope="module")
def pf():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device (there is no CPU fallback to test)")
    import pegaflow_b200

    return pegaflow_b200


def _pair(pf, pool=64 << 20, **kw):
    okw = {}
    if "host_alignment" in kw:
        okw["ssd_alignment"] = kw["host_alignment"]
    if "blockwise_alloc" in kw:
        okw["blockwise_alloc"] = kw["blockwise_alloc"]
    return pf.PegaEngine(pool, **kw), CudaMem(0), OracleEngine(pool, **okw), sc.NumpyMem()


def _compare_images(eng, ora, instance, hashes, n_slots, group=0):
    for h in hashes:
        for slot in range(n_slots):
            a = eng.block_slot_image(instance, h, slot, group)
            b = ora.block_slot_image(instance, h, slot, group)
            assert (a is None) == (b is None)
            if a is not None:
                assert [bytes(x) for x in a] == [bytes(x) for x in b], f"host image of slot {slot} differs"


def _both_roundtrip(pf, layers_spec, save_ids, load_ids, hashes, fills, *, route="auto", n_slots=None, **kw):
    reg = {k: kw.pop(k) for k in list(kw) if k in ("page_first", "use_groups", "use_strides", "one_batch")}
    eng, gmem, ora, nmem = _pair(pf, route=ROUTES[route], min_dma_bytes=64 << 10, **kw)
    try:
        gl = [sc.Layer(**s) for s in layers_spec]
        nl = [sc.Layer(**s) for s in layers_spec]
        got = sc.roundtrip(eng, gmem, "inst", "ns", gl, save_ids, load_ids, hashes, fills=fills, **reg)
        want = sc.roundtrip(ora, nmem, "inst", "ns", nl, save_ids, load_ids, hashes, fills=fills, **reg)
        for L, fill in zip(nl, fills):
            assert np.array_equal(got[L.name], want[L.name]), f"GPU bytes of {L.name} differ from the oracle"
            if not reg.get("page_first"):
                assert np.array_equal(want[L.name], sc.expected_after_roundtrip(L, fill, list(save_ids), list(load_ids)))
        slots = n_slots if n_slots is not None else (1 if reg.get("page_first") else len(gl))
        _compare_images(eng, ora, "inst", hashes, slots)
        m = eng.metrics()
        assert m["load_failures"] == 0 and m["save_batches"] >= 1 and m["load_tasks"] == 1
        return m
    finally:
        eng.close()


def test_save_query_load_roundtrip(pf):
    """engine_basic.rs:12-25."""
    fill = sc.fill_pattern(4, 1024)
    _both_roundtrip(pf, [dict(name="layer_0", num_blocks=4, segment_bytes=1024)], range(4), range(4),
                    sc.make_block_hashes(4, 0), [fill])


@pytest.mark.parametrize("route", list(ROUTES))
def test_page_first_multi_layer_roundtrip(pf, route):
    """engine_basic.rs:32-58: uneven page offsets 0 / 512 / 1536."""
    spec = [dict(name="layer_a", num_blocks=4, segment_bytes=512), dict(name="layer_b", num_blocks=4, segment_bytes=1024),
            dict(name="layer_c", num_blocks=4, segment_bytes=1536)]
    fills = [sc.fill_pattern(4, 512), sc.fill_pattern(4, 1024, 0x40), sc.fill_pattern(4, 1536, 0x80)]
    _both_roundtrip(pf, spec, range(4), [3, 1, 0, 2], sc.make_block_hashes(4, 0xAB), fills, route=route,
                    page_first=True)


@pytest.mark.parametrize("seg,kv_stride,nblocks", [(512, 4096, 4), (4096, 16384, 2)])
def test_split_storage_roundtrip(pf, seg, kv_stride, nblocks):
    """engine_basic.rs:217-252 (both the direct- and the kernel-mode shapes)."""
    L = sc.Layer("layer_0", nblocks, seg, segments=2, kv_stride=kv_stride)
    fill = sc.seeded_bytes(L.region_bytes, 7)
    ids = list(range(nblocks))
    _both_roundtrip(pf, [dict(name="layer_0", num_blocks=nblocks, segment_bytes=seg, segments=2, kv_stride=kv_stride)],
                    ids, ids[::-1], sc.make_block_hashes(nblocks, 1), [fill])


@pytest.mark.parametrize("route", list(ROUTES))
def test_qwen3_kv_layout_roundtrip(pf, route):
    """Qwen3-0.6B shape at reduced layer count: 8 KV heads x 128 x bf16 x 16 tokens = 32 KiB K and V
    regions per layer, 256 GPU blocks, save 64 random ids, load into another random 64."""
    rng = np.random.default_rng(43)
    n_layers, num_blocks, seg = 6, 256, 32768
    spec = [dict(name=f"model.layers.{i}.self_attn.attn", num_blocks=num_blocks, segment_bytes=seg, segments=2,
                 kv_stride=num_blocks * seg) for i in range(n_layers)]
    fills = [rng.standard_normal(2 * num_blocks * seg // 2).astype(np.float16).view(np.uint8) for _ in range(n_layers)]
    save_ids = (rng.permutation(num_blocks - 1)[:64] + 1).tolist()
    load_ids = (rng.permutation(num_blocks - 1)[:64] + 1).tolist()
    m = _both_roundtrip(pf, spec, save_ids, load_ids, sc.make_block_hashes(64, 9), fills, route=route,
                        pool=256 << 20)
    assert m["save_bytes"] == n_layers * 64 * 2 * seg and m["load_bytes"] == m["save_bytes"]


@pytest.mark.parametrize("dtype_bytes", [2, 1])
def test_mla_latent_page_first_roundtrip(pf, dtype_bytes):
    """DeepSeek-style latent cache [num_blocks, 64, 576] (bf16 and fp8 byte widths), page-first pages."""
    rng = np.random.default_rng(44 + dtype_bytes)
    n_layers, num_blocks, seg = 5, 40, 64 * 576 * dtype_bytes
    spec = [dict(name=f"model.layers.{i}.mla", num_blocks=num_blocks, segment_bytes=seg) for i in range(n_layers)]
    fills = [sc.seeded_bytes(num_blocks * seg, 100 + i) for i in range(n_layers)]
    save_ids = (rng.permutation(num_blocks)[:16]).tolist()
    load_ids = (rng.permutation(num_blocks)[:16]).tolist()
    _both_roundtrip(pf, spec, save_ids, load_ids, sc.make_block_hashes(16, 3), fills, page_first=True,
                    pool=128 << 20)


def test_padded_host_strides_and_blockwise_alloc(pf):
    """Host strides padded to 512 bytes (lib.rs:379-388) and one pool allocation per block
    (offload.rs:454-456): the images keep their padding tails untouched."""
    spec = [dict(name="l0", num_blocks=12, segment_bytes=8848), dict(name="l1", num_blocks=12, segment_bytes=1000,
                                                                      segments=2, kv_stride=12 * 1000 + 24)]
    fills = [sc.seeded_bytes(sc.Layer(**s).region_bytes, 3 + i) for i, s in enumerate(spec)]
    ids = [5, 0, 11, 7]
    _both_roundtrip(pf, spec, ids, [1, 2, 3, 4], sc.make_block_hashes(4, 5), fills, host_alignment=512)
    _both_roundtrip(pf, spec, ids, [1, 2, 3, 4], sc.make_block_hashes(4, 5), fills, blockwise_alloc=True)


def test_fused_buffer_block_stride(pf):
    """One layer's view into a buffer that holds all layers of a block (layout.rs:140-153)."""
    spec = [dict(name="fused", num_blocks=8, segment_bytes=8192, block_stride=16384)]
    fill = sc.seeded_bytes(sc.Layer(**spec[0]).region_bytes, 21)
    _both_roundtrip(pf, spec, [7, 2, 5], [0, 1, 6], sc.make_block_hashes(3, 8), [fill], use_strides=True)


def test_hybrid_groups_load_to_distinct_block_ids(pf, kats):
    """engine_basic.rs:62-124 with its spelled-out expected images."""
    eng, mem, _, _ = _pair(pf)
    try:
        layers = [sc.Layer("full_attention", 4, 1024), sc.Layer("gdn", 4, 1024)]
        sc.register(eng, mem, "hyb", "ns", layers, use_groups=True)
        mem.write(layers[0].buf, sc.fill_pattern(4, 1024))
        mem.write(layers[1].buf, sc.fill_pattern(4, 1024, 0x40))
        hashes = sc.make_block_hashes(2, 0xAC)
        eng.batch_save("hyb", 0, 0, 0, [("full_attention", [0, 1], hashes), ("gdn", [2, 3], hashes)])
        eng.flush_saves()
        for L in layers:
            mem.zero(L.buf)
        blocks, missing = eng.query_prefix("hyb", hashes)
        assert missing == 0
        lease = eng.create_query_lease("hyb", blocks)
        eng.batch_load("hyb", 0, 0, [["full_attention"], [], ["gdn"]], [(lease, [[2, 3], [None, None], [None, 0]])])
        full = np.zeros(4096, dtype=np.uint8)
        full[2048:3072] = 1
        full[3072:4096] = 2
        gdn = np.zeros(4096, dtype=np.uint8)
        gdn[0:1024] = kats["engine_roundtrips"]["hybrid_expected"]["gdn"]["0"]
        assert np.array_equal(mem.read(layers[0].buf), full)
        assert np.array_equal(mem.read(layers[1].buf), gdn)
    finally:
        eng.close()


def test_prefix_dedup_and_partial_layer_semantics(pf):
    """engine_basic.rs:165-208 + prefix_semantics.rs."""
    eng, mem, _, _ = _pair(pf)
    try:
        layers = [sc.Layer("layer_0", 4, 1024), sc.Layer("layer_1", 4, 1024)]
        sc.register(eng, mem, "ml", "ns", layers)
        hashes = sc.make_block_hashes(4, 55)
        eng.batch_save("ml", 0, 0, 0, [("layer_0", [0, 1, 2, 3], hashes)])
        eng.flush_saves()
        assert len(eng.query_prefix("ml", hashes)[0]) == 0, "partial save must not expose as hit"
        eng.batch_save("ml", 0, 0, 0, [("layer_1", [0, 1, 2, 3], hashes)])
        eng.flush_saves()
        assert len(eng.query_prefix("ml", hashes)[0]) == 4
        used_before = eng.metrics()["pool_used_bytes"]
        eng.batch_save("ml", 0, 0, 0, [("layer_0", [0, 1, 2, 3], hashes), ("layer_1", [0, 1, 2, 3], hashes)])
        eng.flush_saves()
        assert eng.metrics()["pool_used_bytes"] == used_before, "a save of resident blocks must not allocate"
        # gap breaks the prefix
        gap_layers = [sc.Layer("layer_0", 3, 1024)]      # kept: registered memory must outlive its use
        sc.register(eng, mem, "gap", "ns2", gap_layers)
        allh = sc.make_block_hashes(4, 20)
        eng.batch_save("gap", 0, 0, 0, [("layer_0", [0, 1, 2], [allh[0], allh[2], allh[3]])])
        eng.flush_saves()
        blocks, missing = eng.query_prefix("gap", allh)
        assert (len(blocks), missing) == (1, 3)
        # namespace isolation (engine_basic.rs:255-272)
        assert eng.query_prefix("gap", hashes) == ([], 4)
    finally:
        eng.close()


def test_error_behaviour_matches_the_oracle(pf):
    """The same invalid calls fail with the same variant and text on both engines."""
    eng, gmem, ora, nmem = _pair(pf)
    try:
        def both(fn, match):
            with pytest.raises(pf.PegaFlowError) as e1:
                fn(eng, gmem)
            with pytest.raises(EngineError) as e2:
                fn(ora, nmem)
            assert e1.value.kind == e2.value.kind
            assert match in str(e1.value) and match in str(e2.value)

        both(lambda e, m: e.batch_save("nope", 0, 0, 0, []), "instance nope not found")
        both(lambda e, m: sc.register(e, m, "bad", "ns", [sc.Layer("l", 4, 1024, segments=2, kv_stride=512)]),
             "overlap")
        both(lambda e, m: sc.register(e, m, "bad2", "ns", [sc.Layer("l", 10, 1024, region_bytes=5120)]), "too small")
        keep = []   # registered memory must outlive the engines: the oracle's is plain numpy
        for e, m in ((eng, gmem), (ora, nmem)):
            keep.append([sc.Layer("layer_0", 4, 1024), sc.Layer("layer_1", 4, 1024)])
            sc.register(e, m, "v", "ns", keep[-1])
        both(lambda e, m: sc.register(e, m, "v", "ns", [sc.Layer("layer_0", 4, 1024)]), "already exists")
        both(lambda e, m: sc.register(e, m, "v", "ns", [sc.Layer("layer_0", 4, 1024)], device_id=1),
             "already fully registered")
        both(lambda e, m: sc.register(e, m, "v", "ns", [sc.Layer("layer_0", 4, 1024)], tp_size=2), "topology mismatch")
        both(lambda e, m: e.batch_save("v", 0, 0, 0, [("layer_0", [4], [b"h"])]), "block_id 4 out of range")
        both(lambda e, m: e.batch_save("v", 0, 0, 0, [("layer_0", [1, 2], [b"h"])]), "does not match block_hashes")
        both(lambda e, m: e.batch_save("v", 0, 0, 9, [("layer_0", [1], [b"h"])]), "device 9 not found")
        both(lambda e, m: e.batch_save("v", 1, 0, 0, [("layer_0", [1], [b"h"])]), "but save requested")
        both(lambda e, m: e.batch_save("v", 0, 0, 0, [("layer_x", [1], [b"h"])]), "layer layer_x is not registered")
        both(lambda e, m: e.create_query_lease("v", []), "requires at least one block")
        both(lambda e, m: e.batch_load("v", 0, 0, [], []), "at least one layer group")
        both(lambda e, m: e.batch_load("v", 0, 0, [["layer_0"], ["layer_0"]], []), "unique across groups")
        both(lambda e, m: e.batch_load("v", 0, 0, [["layer_0"]], [(b"\0" * 16, [[0]])]), "unknown or expired")
        # page-first partial save (engine_basic.rs:131-158)
        for e, m in ((eng, gmem), (ora, nmem)):
            keep.append([sc.Layer(n, 4, 512) for n in ("layer_a", "layer_b", "layer_c")])
            sc.register(e, m, "pf", "ns3", keep[-1],
                        page_first=True)
        both(lambda e, m: e.batch_save("pf", 0, 0, 0, [("layer_a", [0, 1, 2, 3], sc.make_block_hashes(4, 0xCD))]),
             "must cover all")
        # lease accounting: world_size consumers, then gone (lease.rs:98-133)
        h = sc.make_block_hashes(2, 77)
        for e in (eng, ora):
            e.batch_save("v", 0, 0, 0, [("layer_0", [0, 1], h), ("layer_1", [0, 1], h)])
            e.flush_saves()
            blocks, missing = e.query_prefix("v", h)
            assert missing == 0
            lease = e.create_query_lease("v", blocks)
            e.batch_load("v", 0, 0, [["layer_0", "layer_1"]], [(lease, [[2, 3]])])
            assert e.release_query_lease(lease) is False
            lease2 = e.create_query_lease("v", blocks)
            assert e.release_query_lease(lease2) is True
        both(lambda e, m: e.unregister_instance("ghost"), "instance ghost not found")
    finally:
        eng.close()


def test_pool_exhaustion_evicts_lru_then_fails(pf):
    """storage/mod.rs:294-330: a full pool evicts least recently used blocks; a request larger
    than the pool fails with the reference's message and counts an allocation failure."""
    eng = pf.PegaEngine(1 << 20)
    mem = CudaMem(0)
    try:
        L = sc.Layer("layer_0", 64, 65536)
        sc.register(eng, mem, "ev", "ns", [L])
        mem.write(L.buf, sc.seeded_bytes(L.region_bytes, 1))
        first = sc.make_block_hashes(8, 1)
        eng.batch_save("ev", 0, 0, 0, [("layer_0", list(range(8)), first)])     # 512 KiB
        eng.flush_saves()
        second = sc.make_block_hashes(12, 2)
        eng.batch_save("ev", 0, 0, 0, [("layer_0", list(range(8, 20)), second)])  # 768 KiB: must evict
        eng.flush_saves()
        m = eng.metrics()
        assert m["evicted_blocks"] >= 8 and len(eng.query_prefix("ev", second)[0]) == 12
        assert len(eng.query_prefix("ev", first)[0]) == 0
        with pytest.raises(pf.PegaflowInternal, match="pinned pool exhausted while allocating block buffer"):
            eng.batch_save("ev", 0, 0, 0, [("layer_0", list(range(20, 40)), sc.make_block_hashes(20, 3))])
        assert eng.metrics()["pool_alloc_failures"] == 1
    finally:
        eng.close()


def _eviction_env(pf, instance, **kw):
    """tests/eviction.rs:12-25: one layer of 4 blocks x 4096 bytes, a pool that holds two batches."""
    eng = pf.PegaEngine(4 * 4096 * 2, enable_numa_affinity=False, **kw)
    mem = CudaMem(0)
    L = sc.Layer("layer_0", 4, 4096)
    sc.register(eng, mem, instance, "ns-evict", [L])
    return eng, mem, L


def _load_and_read(eng, mem, L, instance, lease, n):
    mem.zero(L.buf)
    eng.batch_load(instance, 0, 0, [["layer_0"]], [(lease, [list(range(n))])])
    mem.sync()
    return mem.read(L.buf)


@pytest.mark.parametrize("shards", [1, 2])
def test_eviction_reclaims_old_blocks_for_new(pf, shards):
    """tests/eviction.rs:27-49 and :84-107 (the same with pool_shards = 2): blocks saved after the GPU
    data was overwritten load the overwritten data, whatever had to be evicted for them."""
    eng, mem, L = _eviction_env(pf, "inst-evict", pool_shards=shards)
    try:
        mem.write(L.buf, sc.fill_pattern(4, 4096))
        eng.batch_save("inst-evict", 0, 0, 0, [("layer_0", [0, 1, 2, 3], sc.make_block_hashes(4, 1))])
        eng.flush_saves()
        fresh = sc.fill_pattern(4, 4096, delta=42)
        mem.write(L.buf, fresh)
        new = sc.make_block_hashes(4, 2)
        eng.batch_save("inst-evict", 0, 0, 0, [("layer_0", [0, 1, 2, 3], new)])
        eng.flush_saves()
        third = sc.make_block_hashes(4, 3)
        eng.batch_save("inst-evict", 0, 0, 0, [("layer_0", [0, 1, 2, 3], third)])   # cannot fit without eviction
        eng.flush_saves()
        assert eng.metrics()["evicted_blocks"] >= 1
        for hashes in (new, third):
            blocks, missing = eng.query_prefix("inst-evict", hashes)
            if missing:
                continue   # this batch was the one reclaimed
            got = _load_and_read(eng, mem, L, "inst-evict", eng.create_query_lease("inst-evict", blocks), 4)
            assert np.array_equal(got, fresh)
        assert eng.query_prefix("inst-evict", third)[1] == 0
    finally:
        eng.close()


def test_leased_blocks_survive_eviction_pressure(pf):
    """tests/eviction.rs:51-81: a query lease pins its blocks' memory and their cache entries; pressure
    reclaims the unleased batch instead."""
    eng, mem, L = _eviction_env(pf, "inst-lease")
    try:
        fill = sc.fill_pattern(4, 4096)
        mem.write(L.buf, fill)
        hashes = sc.make_block_hashes(4, 10)
        eng.batch_save("inst-lease", 0, 0, 0, [("layer_0", [0, 1, 2, 3], hashes)])
        eng.flush_saves()
        blocks, missing = eng.query_prefix("inst-lease", hashes)
        assert missing == 0
        lease = eng.create_query_lease("inst-lease", blocks)
        del blocks    # the lease alone pins them from here on
        reclaimed = sc.make_block_hashes(4, 20)
        eng.batch_save("inst-lease", 0, 0, 0, [("layer_0", [0, 1, 2, 3], reclaimed)])
        eng.flush_saves()
        pressure = sc.make_block_hashes(4, 21)
        eng.batch_save("inst-lease", 0, 0, 0, [("layer_0", [0, 1, 2, 3], pressure)])
        eng.flush_saves()
        assert len(eng.query_prefix("inst-lease", reclaimed)[0]) == 0
        again, missing = eng.query_prefix("inst-lease", hashes)
        assert missing == 0 and len(again) == 4
        second = eng.create_query_lease("inst-lease", again)
        del again
        assert eng.release_query_lease(second) is True
        got = _load_and_read(eng, mem, L, "inst-lease", lease, 4)
        assert np.array_equal(got, fill)
    finally:
        eng.close()


def test_stale_inflight_blocks_are_swept_and_their_memory_returned(pf):
    """lib.rs:938-948: blocks that wait for slots which never come (here: the second layer is never saved) are
    dropped by the sweep once they are older than the age given, and nothing younger is."""
    import time

    eng, mem, _, _ = _pair(pf)
    try:
        layers = [sc.Layer("layer_0", 4, 1024), sc.Layer("layer_1", 4, 1024)]
        sc.register(eng, mem, "gc", "ns", layers)
        assert eng.gc_stale_inflight(0.0) == 0
        hashes = sc.make_block_hashes(4, 77)
        eng.batch_save("gc", 0, 0, 0, [("layer_0", [0, 1, 2, 3], hashes)])
        eng.flush_saves()
        assert len(eng.query_prefix("gc", hashes)[0]) == 0 and eng.metrics()["pool_used_bytes"] > 0
        assert eng.gc_stale_inflight(300.0) == 0, "a block younger than the age limit was swept"
        time.sleep(0.05)
        assert eng.gc_stale_inflight(0.01) == 4
        assert eng.metrics()["pool_used_bytes"] == 0 and eng.gc_stale_inflight(0.0) == 0
        # the same blocks can be saved again, completely this time
        eng.batch_save("gc", 0, 0, 0, [("layer_0", [0, 1, 2, 3], hashes), ("layer_1", [0, 1, 2, 3], hashes)])
        eng.flush_saves()
        assert len(eng.query_prefix("gc", hashes)[0]) == 4
        with pytest.raises(pf.PegaFlowError, match="max_age_seconds"):
            eng.gc_stale_inflight(-1.0)
    finally:
        eng.close()


def test_instance_listing_namespace_and_unregister_all(pf):
    """lib.rs:459-489: list_instance_ids, instance_namespace, unregister_all_instances."""
    eng = pf.PegaEngine(4 << 20, enable_numa_affinity=False)
    mem = CudaMem(0)
    try:
        assert eng.list_instance_ids() == [] and eng.unregister_all_instances() == []
        layers = []
        for name, ns in (("inst-b", "ns-1"), ("inst-a", "ns-2")):
            L = sc.Layer("layer_0", 4, 4096)
            layers.append(L)
            sc.register(eng, mem, name, ns, [L])
        assert eng.list_instance_ids() == ["inst-a", "inst-b"]
        assert eng.instance_namespace("inst-a") == "ns-2" and eng.instance_namespace("inst-b") == "ns-1"
        with pytest.raises(pf.PegaFlowError, match="instance nobody not found"):
            eng.instance_namespace("nobody")
        h = sc.make_block_hashes(2, 40)
        eng.batch_save("inst-a", 0, 0, 0, [("layer_0", [0, 1], h)])
        eng.flush_saves()
        blocks, _ = eng.query_prefix("inst-a", h)
        lease = eng.create_query_lease("inst-a", blocks)
        del blocks
        assert eng.unregister_all_instances() == ["inst-a", "inst-b"]
        assert eng.list_instance_ids() == [] and eng.release_query_lease(lease) is False   # leases went with the instances
        with pytest.raises(pf.PegaFlowError, match="instance inst-a not found"):
            eng.batch_save("inst-a", 0, 0, 0, [("layer_0", [0, 1], h)])
    finally:
        eng.close()


def test_cleanup_memory_cache_drops_every_resident_block(pf):
    """storage/mod.rs:395-445 and its test (:662-681): every resident block leaves the cache; the ones a lease
    still holds are counted as still referenced and keep their pool memory until the lease has been used or
    released; a second clean-up finds nothing."""
    eng, mem, L = _eviction_env(pf, "inst-clean")
    try:
        fill = sc.fill_pattern(4, 4096)
        mem.write(L.buf, fill)
        held, free = sc.make_block_hashes(2, 30), sc.make_block_hashes(2, 31)
        eng.batch_save("inst-clean", 0, 0, 0, [("layer_0", [0, 1], held)])      # two saves: two pool allocations
        eng.batch_save("inst-clean", 0, 0, 0, [("layer_0", [2, 3], free)])
        eng.flush_saves()
        used = eng.metrics()["pool_used_bytes"]
        assert used > 0 and eng.metrics()["cache_blocks"] == 4
        blocks, missing = eng.query_prefix("inst-clean", held)
        assert missing == 0
        lease = eng.create_query_lease("inst-clean", blocks)
        del blocks
        stats = eng.cleanup_memory_cache()
        assert stats["evicted_blocks"] == 4 and stats["still_referenced_blocks"] == 2
        assert stats["evicted_bytes"] == 4 * 4096 and stats["reclaimed_bytes"] == used // 2
        m = eng.metrics()
        assert m["cache_blocks"] == 0 and m["pool_used_bytes"] == used - stats["reclaimed_bytes"]
        assert len(eng.query_prefix("inst-clean", held)[0]) == 0 and len(eng.query_prefix("inst-clean", free)[0]) == 0
        assert eng.cleanup_memory_cache() == {"evicted_blocks": 0, "evicted_bytes": 0, "reclaimed_bytes": 0,
                                              "still_referenced_blocks": 0}
        # the lease still loads what it pinned, and its memory goes back once it has been consumed
        got = _load_and_read(eng, mem, L, "inst-clean", lease, 2)
        assert np.array_equal(got[:2 * 4096], fill[:2 * 4096])
        import time

        deadline = time.time() + 5          # the load task lets go of its blocks just after it has reported
        while eng.metrics()["pool_used_bytes"] and time.time() < deadline:
            time.sleep(0.01)
        assert eng.metrics()["pool_used_bytes"] == 0
    finally:
        eng.close()


def test_load_state_shm_completion_and_failure(pf):
    """lib.rs:654-680 + sync_state.rs: a cross-process style load completes through the
    shared-memory word; a pre-submit error flips it to ERROR."""
    import time

    eng = pf.PegaEngine(16 << 20)
    mem = CudaMem(0)
    try:
        L = sc.Layer("layer_0", 8, 4096)
        sc.register(eng, mem, "shm", "ns", [L])
        fill = sc.seeded_bytes(L.region_bytes, 9)
        mem.write(L.buf, fill)
        h = sc.make_block_hashes(8, 4)
        eng.batch_save("shm", 0, 0, 0, [("layer_0", list(range(8)), h)])
        eng.flush_saves()
        mem.zero(L.buf)
        blocks, _ = eng.query_prefix("shm", h)
        state = pf.PyLoadState()
        assert state.get_state() == 0 and state.shm_name().startswith("pega_load_")
        eng.batch_load_shm("shm", 0, 0, state.shm_name(), [["layer_0"]],
                           [(eng.create_query_lease("shm", blocks), [list(range(8))])])
        deadline = time.time() + 5
        while not state.is_ready() and time.time() < deadline:
            time.sleep(0.001)
        assert state.get_state() == 1
        assert np.array_equal(mem.read(L.buf), fill)
        bad = pf.PyLoadState()
        with pytest.raises(pf.PegaFlowError):
            eng.batch_load_shm("shm", 0, 0, bad.shm_name(), [["layer_0"]], [(b"\1" * 16, [[0]])])
        assert bad.get_state() == -1
        with pytest.raises(pf.PegaflowInternal, match="LoadState"):
            eng.batch_load_shm("shm", 0, 0, "pega_load_does_not_exist", [["layer_0"]], [])
    finally:
        eng.close()


def test_layerwise_async_save_and_per_layer_load_events(pf):
    """Layer-wise pipeline: layers saved one by one as a compute stream produces them, and a
    consumer stream that waits on each layer's load event before touching the layer."""
    import torch

    eng = pf.PegaEngine(64 << 20, min_dma_bytes=64 << 10)
    mem = CudaMem(0)
    try:
        n_layers, num_blocks, seg = 4, 32, 16384
        layers = [sc.Layer(f"l{i}", num_blocks, seg, segments=2, kv_stride=num_blocks * seg) for i in range(n_layers)]
        sc.register(eng, mem, "lw", "ns", layers)
        compute = torch.cuda.Stream()
        ids = list(range(1, 17))
        h = sc.make_block_hashes(16, 6)
        fills, ready_events = [], []
        for i, L in enumerate(layers):
            fill = torch.from_numpy(sc.seeded_bytes(L.region_bytes, 50 + i)).pin_memory()
            fills.append(fill)
            with torch.cuda.stream(compute):
                L.buf.copy_(fill, non_blocking=True)      # stands in for the layer's attention writing its KV
                ready = make_event(torch)
                ready.record(compute)
            ready_events.append(ready)                    # must outlive the save that waits on it
            eng.save_layers_async("lw", 0, 0, 0, [(L.name, ids, h)], ready.cuda_event)
        eng.flush_saves()
        blocks, missing = eng.query_prefix("lw", h)
        assert missing == 0
        compute.synchronize()
        for L in layers:
            mem.zero(L.buf)
        dst = list(range(16, 32))
        done = eng.batch_load_async("lw", 0, 0, [[L.name for L in layers]],
                                    [(eng.create_query_lease("lw", blocks), [dst])])
        outs = []
        for L in layers:
            ev = eng.layer_load_event("lw", 0, L.name)
            eng.stream_wait_event(compute.cuda_stream, ev)
            with torch.cuda.stream(compute):
                outs.append(L.buf.clone())               # the layer's consumer
        compute.synchronize()
        assert done.wait(10) == 1
        for L, fill, out in zip(layers, fills, outs):
            want = sc.expected_after_roundtrip(L, fill.numpy(), ids, dst)
            assert np.array_equal(out.cpu().numpy(), want), "consumer ran before the layer's bytes had landed"
    finally:
        eng.close()


@pytest.mark.parametrize("route", list(ROUTES))
def test_saves_and_loads_running_at_once_stay_bit_exact(pf, route):
    """The save worker and the load worker of one GPU run at the same time (gpu_worker.rs:161-262 gives
    each its own thread and stream): a request's blocks are saved from one thread while another
    request's stored blocks are loaded into different block ids; both results are checked byte for byte."""
    import threading

    eng = pf.PegaEngine(256 << 20, route=ROUTES[route], min_dma_bytes=64 << 10)
    mem = CudaMem(0)
    try:
        n_layers, num_blocks, seg = 4, 512, 16384
        layers = [sc.Layer(f"l{i}", num_blocks, seg, segments=2, kv_stride=num_blocks * seg) for i in range(n_layers)]
        sc.register(eng, mem, "dx", "ns", layers)
        fills = [sc.seeded_bytes(L.region_bytes, 300 + i) for i, L in enumerate(layers)]
        for L, f in zip(layers, fills):
            mem.write(L.buf, f)
        rng = np.random.default_rng(77)
        perm = (rng.permutation(num_blocks - 1) + 1).tolist()
        first, dst = perm[:96], perm[96:192]
        rounds = [perm[192 + 96 * k: 192 + 96 * (k + 1)] for k in range(3)]
        h_first = sc.make_block_hashes(96, 40)
        eng.batch_save("dx", 0, 0, 0, [(L.name, first, h_first) for L in layers])
        eng.flush_saves()
        blocks, missing = eng.query_prefix("dx", h_first)
        assert missing == 0
        names = [L.name for L in layers]
        for k, ids in enumerate(rounds):
            hk = sc.make_block_hashes(96, 41 + k)
            errors = []

            def saver():
                try:
                    eng.batch_save("dx", 0, 0, 0, [(L.name, ids, hk) for L in layers])
                except Exception as e:   # surfaced below, on the test's thread
                    errors.append(e)

            t = threading.Thread(target=saver)
            done = eng.batch_load_async("dx", 0, 0, [names], [(eng.create_query_lease("dx", blocks), [dst])])
            t.start()
            assert done.wait(20) == 1
            t.join()
            assert not errors, errors
            eng.flush_saves()
            mem.sync()
            for li, (L, f) in enumerate(zip(layers, fills)):
                got = mem.read(L.buf)
                want = f.copy()
                loaded = sc.expected_after_roundtrip(L, f, first, dst)
                for d in dst:
                    for off in (0, L.kv_stride):
                        want[off + d * seg: off + (d + 1) * seg] = loaded[off + d * seg: off + (d + 1) * seg]
                assert np.array_equal(got, want), f"round {k}: {L.name} differs after a load that overlapped a save"
                for j in (0, 47, 95):
                    img = eng.block_slot_image("dx", hk[j], li)
                    assert img is not None
                    b = ids[j]
                    assert [bytes(x) for x in img] == [bytes(f[off + b * seg: off + (b + 1) * seg])
                                                       for off in (0, L.kv_stride)]
            for L, f in zip(layers, fills):   # the destinations get their own bytes back for the next round
                mem.write(L.buf, f)
        assert eng.metrics()["load_failures"] == 0
    finally:
        eng.close()


def test_recurrent_group_seals_final_block_save(pf):
    """tests/hybrid_groups.rs:16-178 and :180-217, replayed on the CUDA engine and on the oracle model:
    an attention group saves every block, the recurrent group only a tail checkpoint; membership is per
    group; one load with two leases restores the attention prefix and the checkpoint into another slot."""
    eng, gmem, ora, nmem = _pair(pf)
    try:
        results = []
        for e, m in ((eng, gmem), (ora, nmem)):
            layers = [sc.Layer("attn_0", 8, 1024, group=0), sc.Layer("attn_1", 8, 1024, group=0),
                      sc.Layer("recurrent_state", 8, 2048, group=1)]
            sc.register(e, m, "hybrid-hma", "hybrid-hma-ns", layers, use_groups=True)
            fills = [sc.seeded_bytes(L.region_bytes, 60 + i) for i, L in enumerate(layers)]
            for L, f in zip(layers, fills):
                m.write(L.buf, f)
            hashes = sc.make_block_hashes(8, 10)
            prefix = hashes[:3]
            e.batch_save("hybrid-hma", 0, 0, 0, [("attn_0", [0, 1, 2], prefix), ("attn_1", [0, 1, 2], prefix)])
            e.batch_save("hybrid-hma", 0, 0, 0, [("recurrent_state", [5], [hashes[2]])])
            e.flush_saves()
            attn_hits = e.query_group_membership("hybrid-hma", 0, prefix)
            assert [b is not None for b in attn_hits] == [True, True, True]
            recur_hits = e.query_group_membership("hybrid-hma", 1, prefix)
            assert [b is not None for b in recur_hits] == [False, False, True]
            blocks, missing = e.query_prefix("hybrid-hma", prefix)
            assert len(blocks) == 3 and missing == 0
            attn_lease = e.create_query_lease("hybrid-hma", blocks)
            recur_lease = e.create_query_lease("hybrid-hma", [recur_hits[2]])
            for L in layers:
                m.zero(L.buf)
            e.batch_load("hybrid-hma", 0, 0, [["attn_0", "attn_1"], ["recurrent_state"]],
                         [(attn_lease, [[0, 1, 2], [None, None, None]]), (recur_lease, [[None], [7]])])
            m.sync()
            got = [m.read(L.buf) for L in layers]
            for g, f in zip(got[:2], fills[:2]):
                want = np.zeros_like(f)
                want[:3 * 1024] = f[:3 * 1024]
                assert np.array_equal(g, want)
            want = np.zeros_like(fills[2])
            want[7 * 2048:8 * 2048] = fills[2][5 * 2048:6 * 2048]
            assert np.array_equal(got[2], want)
            results.append(got)
        for a, b in zip(*results):
            assert np.array_equal(a, b)

        # single-group instances: group 0 behaves as before, any other group is an error, not a miss
        for e, m in ((eng, gmem), (ora, nmem)):
            layers = [sc.Layer("layer_0", 4, 1024), sc.Layer("layer_1", 4, 1024)]
            sc.register(e, m, "hybrid-compat", "hybrid-compat-ns", layers)
            for L in layers:
                m.write(L.buf, sc.fill_pattern(4, 1024))
            h = sc.make_block_hashes(4, 7)
            e.batch_save("hybrid-compat", 0, 0, 0, [(L.name, [0, 1], h[:2]) for L in layers])
            e.flush_saves()
            hits = e.query_group_membership("hybrid-compat", 0, h)
            assert [b is not None for b in hits] == [True, True, False, False]
        with pytest.raises(pf.PegaFlowError) as e1:
            eng.query_group_membership("hybrid-compat", 7, h[:1])
        with pytest.raises(EngineError) as e2:
            ora.query_group_membership("hybrid-compat", 7, h[:1])
        assert e1.value.kind == e2.value.kind
    finally:
        eng.close()


def test_query_lease_protocol_and_stateless_queries(pf):
    """tests/prefetch_lease.rs:11-27 (a released lease cannot be loaded) and prefix_semantics.rs:86-126
    (a miss does not hide blocks saved later under the same request id; an empty query is zero / zero)."""
    eng, gmem, ora, nmem = _pair(pf)
    try:
        for e, m in ((eng, gmem), (ora, nmem)):
            L = sc.Layer("layer_0", 4, 1024)
            sc.register(e, m, "lease-proto", "test-ns", [L])
            m.write(L.buf, sc.fill_pattern(4, 1024))
            h = sc.make_block_hashes(4, 40)
            blocks, missing = e.query_prefix("lease-proto", h)
            assert len(blocks) == 0 and missing == 4
            e.batch_save("lease-proto", 0, 0, 0, [("layer_0", [0, 1, 2, 3], h)])
            e.flush_saves()
            blocks, missing = e.query_prefix("lease-proto", h)
            assert len(blocks) == 4 and missing == 0
            blocks0, missing0 = e.query_prefix("lease-proto", [])
            assert len(blocks0) == 0 and missing0 == 0
            lease = e.create_query_lease("lease-proto", blocks)
            assert e.release_query_lease(lease) is True
            with pytest.raises((pf.PegaFlowError, EngineError), match="query lease is unknown or expired"):
                e.batch_load("lease-proto", 0, 0, [["layer_0"]], [(lease, [[0, 1, 2, 3]])])
    finally:
        eng.close()
