"""Pin the CPU oracle to the reference's own known-answer tests (no GPU needed)."""
import json
import os

import numpy as np
import pytest

from oracle import pf_oracle as po

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _make_layout(case):
    lay = po.KVCacheLayout(*case["new"])
    if "block_stride" in case:
        lay.with_block_stride(case["block_stride"])
    if "ssd_padding" in case:
        lay.with_ssd_padding(case["ssd_padding"])
    return lay


def test_layout_known_answers(kats):
    for case in kats["layout"]["ok"]:
        lay = _make_layout(case)
        if "split" in case:
            assert lay.is_split == case["split"], case["name"]
        for idx, want in case.get("copies", {}).items():
            assert lay.block_copies(int(idx)) == [tuple(x) for x in want], case["name"]
        for idx in case.get("out_of_range", []):
            with pytest.raises(po.OracleError, match="out of range"):
                lay.block_copies(idx)
        for key in ("padded_segment_bytes", "padded_block_bytes"):
            if key in case:
                assert getattr(lay, key) == case[key], case["name"]


def test_layout_rejects(kats):
    for case in kats["layout"]["reject"]:
        with pytest.raises(po.OracleError) as ei:
            _make_layout(case)
        assert case["contains"] in str(ei.value), (case["name"], str(ei.value))


def test_page_layout_known_answers(kats):
    for case in kats["page_layout"]["ok"]:
        got = po.build_page_layout(case["sets"], case["n_layers"], case["padded"])
        for key in ("shard_page_sizes", "layer_shard", "layer_offsets", "layer_bytes"):
            assert got[key] == case[key], (case["name"], key)
    for case in kats["page_layout"]["reject"]:
        with pytest.raises(po.OracleError) as ei:
            po.build_page_layout(case["sets"], case["n_layers"], case["padded"])
        assert case["contains"] in str(ei.value)


def test_merge_rule(kats):
    for case in kats["merge"]["cases"]:
        n = len(case["descs"])
        arr = (po.CopyDesc * n)()
        for i, (dev, host, size, da, ha) in enumerate(case["descs"]):
            arr[i] = po.CopyDesc(dev, host, 0, size, da, ha)
        out, m = po.merge(arr, n)
        assert [[out[i].device, out[i].host, out[i].size] for i in range(m)] == case["merged"]


def test_unit_size(kats):
    for case in kats["allocator"]["unit_size"]:
        assert po.pool_unit_size(case["pool"], case["hint"]) == case["unit"]


def test_group_hash(kats):
    for case in kats["group_hash"]["cases"]:
        assert po.group_hash(bytes(case["hash"]), case["group"]) == bytes(case["out"])


def test_load_state_image(kats):
    ls = kats["load_state"]
    img = po.load_state_image()
    assert len(img) == ls["mapping_bytes"]
    assert int.from_bytes(img[:8], "little") == ls["offset_word"]
    assert int.from_bytes(img[8:12], "little") == ls["magic"]
    assert int.from_bytes(img[12:16], "little") == ls["version"]
    assert po.parse_load_state(img) == ls["pending"]
    assert po.parse_load_state(po.load_state_image(1)) == ls["success"]
    assert po.parse_load_state(po.load_state_image(-1)) == ls["error"]
    with pytest.raises(po.OracleError, match="too small"):
        po.parse_load_state(b"\0")
    bad = bytearray(img)
    bad[8:12] = (0xDEADBEEF).to_bytes(4, "little")
    with pytest.raises(po.OracleError, match="invalid LoadState header"):
        po.parse_load_state(bytes(bad))


def test_layout_inference_matches_reference_fixture():
    with open(os.path.join(GOLDEN, "kv_layout_inference.json")) as f:
        fx = json.load(f)
    assert len(fx["cases"]) > 300
    for c in fx["cases"]:
        kw = dict(is_mla=c["is_mla"], is_recurrent_state=c["is_recurrent_state"])
        if "error" in c:
            with pytest.raises(ValueError) as ei:
                po.infer_kv_cache_registration(c["shape"], c["stride"], c["element_size"], c["logical_block_size"], **kw)
            assert str(ei.value) == c["error"]
        else:
            got = po.infer_kv_cache_registration(c["shape"], c["stride"], c["element_size"],
                                                 c["logical_block_size"], **kw)
            assert got == c["result"], c


def test_kernel_roundtrip_pattern_both_directions(kats):
    """transfer/kernel.rs:205-267 replayed on the oracle: 257 x 4112-byte segments."""
    k = kats["kernel_roundtrip"]
    n, seg = k["segments"], k["segment_bytes"]
    total = n * seg
    pattern = ((np.arange(total, dtype=np.uint64) * 31 + 7) & 0xFF).astype(np.uint8)
    dev = np.zeros(total, dtype=np.uint8)
    host = pattern.copy()
    descs = (po.CopyDesc * n)()
    for i in range(n):
        descs[i] = po.CopyDesc(dev.ctypes.data + i * seg, host.ctypes.data + i * seg, host.ctypes.data + i * seg, seg, 0, 0)
    po.execute(descs, n, host_is_src=True)
    assert np.array_equal(dev, pattern)
    host[:] = 0
    po.execute(descs, n, host_is_src=False, threads=4)
    assert np.array_equal(host, pattern)


def test_build_copy_descs_pairs_k_and_v():
    """gpu_worker.rs:353-423: split block, two host segments vs one host segment."""
    lay = po.KVCacheLayout(0x1000, 200 * 1024, 100, 1024, 100 * 1024, 2)
    two = [(3, [po.HostSeg(0x9000, 0xA9000, 7), po.HostSeg(0x20000, 0xB0000, 8)], 0)]
    d, n, total = po.build_copy_descs([(lay, two)])
    assert n == 2 and total == 2048
    assert d[0].as_tuple() == (0x1000 + 3 * 1024, 0x9000, 0xA9000, 1024, 0, 7)
    assert d[1].as_tuple() == (0x1000 + 103 * 1024, 0x20000, 0xB0000, 1024, 0, 8)
    one = [(3, [po.HostSeg(0x9000, 0xA9000, 7)], 512)]
    d, n, total = po.build_copy_descs([(lay, []), (lay, one)])
    assert n == 2
    assert d[0].as_tuple() == (0x1000 + 3 * 1024, 0x9000 + 512, 0xA9000 + 512, 1024, 1, 7)
    assert d[1].as_tuple() == (0x1000 + 103 * 1024, 0x9000 + 512 + 1024, 0xA9000 + 512 + 1024, 1024, 1, 7)
    with pytest.raises(po.OracleError, match="out of range"):
        po.build_copy_descs([(lay, [(100, [po.HostSeg(1, 1, 1)], 0)])])
