"""Engine round-trip scenarios shared by the oracle tests (CPU) and the CUDA parity tests.

Every scenario drives an engine object through the same public calls the reference's own
integration tests make (pegaflow-core/tests/engine_basic.rs, tests/common/harness.rs):
register -> save -> wipe GPU -> prefix query -> lease -> load -> compare.  ``mem`` abstracts
where "GPU memory" lives (numpy for the oracle, a CUDA buffer for the product).
"""
from __future__ import annotations

import numpy as np


def make_block_hashes(n, salt):
    """tests/common/helpers.rs:91-100: salt byte + little-endian u32 index."""
    return [bytes([salt]) + int(i).to_bytes(4, "little") for i in range(n)]


def fill_pattern(nblocks, block_bytes, delta=0):
    """tests/common/helpers.rs:79-89 (+ gpu_buffer overwrite): block i = byte (i % 251) + 1 (+ delta)."""
    a = np.empty((nblocks, block_bytes), dtype=np.uint8)
    for i in range(nblocks):
        a[i, :] = ((i % 251) + 1 + delta) & 0xFF
    return a.reshape(-1)


def seeded_bytes(n, seed):
    return np.random.default_rng(seed).integers(0, 256, size=n, dtype=np.uint8)


class Layer:
    def __init__(self, name, num_blocks, segment_bytes, *, segments=1, kv_stride=0, block_stride=None, group=0,
                 region_bytes=None):
        self.name, self.num_blocks, self.segment_bytes = name, num_blocks, segment_bytes
        self.segments, self.kv_stride, self.block_stride, self.group = segments, kv_stride, block_stride, group
        if region_bytes is None:
            if segments == 2 and kv_stride > segment_bytes:
                stride = block_stride or segment_bytes
                region_bytes = kv_stride + (num_blocks - 1) * stride + segment_bytes
            else:
                stride = block_stride or segment_bytes * segments
                region_bytes = (num_blocks - 1) * stride + segment_bytes * segments
        self.region_bytes = region_bytes
        self.buf = None  # set by the memory backend


def register(engine, mem, instance_id, namespace, layers, *, device_id=0, tp_rank=0, pp_rank=0, tp_size=1,
             world_size=1, transfer_mode="direct", page_first=False, use_groups=False, use_strides=False):
    for L in layers:
        if L.buf is None:
            L.buf = mem.alloc(L.region_bytes)
    engine.register_context_layer_batch_strided(
        instance_id, namespace, device_id, tp_rank, pp_rank, tp_size, world_size,
        [L.name for L in layers], [mem.ptr(L.buf) for L in layers], [L.region_bytes for L in layers],
        [L.num_blocks for L in layers], [L.segment_bytes for L in layers], [L.kv_stride for L in layers],
        [L.segments for L in layers],
        [L.block_stride or (L.segment_bytes if (L.segments == 2 and L.kv_stride > L.segment_bytes)
                            else L.segment_bytes * L.segments) for L in layers] if use_strides else None,
        [L.group for L in layers] if use_groups else None,
        transfer_mode, page_first)


class NumpyMem:
    """"GPU memory" for the oracle: plain numpy buffers."""

    def alloc(self, nbytes):
        return np.zeros(nbytes, dtype=np.uint8)

    def ptr(self, buf):
        return buf.ctypes.data

    def write(self, buf, data):
        buf[:] = data

    def read(self, buf):
        return buf.copy()

    def zero(self, buf):
        buf[:] = 0

    def sync(self):
        pass


def roundtrip(engine, mem, instance_id, namespace, layers, save_ids, load_ids, hashes, *, fills, page_first=False,
              one_batch=True, **reg):
    """Save ``save_ids`` of every layer under ``hashes``, wipe, load them into ``load_ids``.

    Returns {layer_name: bytes after load} so two engines can be compared."""
    register(engine, mem, instance_id, namespace, layers, page_first=page_first, **reg)
    for L, fill in zip(layers, fills):
        mem.write(L.buf, fill)
    saves = [(L.name, list(save_ids), list(hashes)) for L in layers]
    if one_batch:
        engine.batch_save(instance_id, reg.get("tp_rank", 0), reg.get("pp_rank", 0), reg.get("device_id", 0), saves)
    else:
        for s in saves:
            engine.batch_save(instance_id, reg.get("tp_rank", 0), reg.get("pp_rank", 0), reg.get("device_id", 0), [s])
    engine.flush_saves()
    for L in layers:
        mem.zero(L.buf)
    blocks, missing = engine.query_prefix(instance_id, hashes)
    assert missing == 0 and len(blocks) == len(hashes)
    lease = engine.create_query_lease(instance_id, blocks)
    engine.batch_load(instance_id, reg.get("tp_rank", 0), reg.get("device_id", 0), [[L.name for L in layers]],
                      [(lease, [list(load_ids)])])
    mem.sync()
    return {L.name: mem.read(L.buf) for L in layers}


def expected_after_roundtrip(layer: Layer, fill, save_ids, load_ids):
    """What a layer must hold after save(save_ids) -> zero -> load(load_ids): independent of any engine."""
    out = np.zeros(layer.region_bytes, dtype=np.uint8)
    split = layer.segments == 2 and layer.kv_stride > layer.segment_bytes
    stride = layer.block_stride or (layer.segment_bytes if split else layer.segment_bytes * layer.segments)
    for s, d in zip(save_ids, load_ids):
        if d is None:
            continue
        if split:
            for off in (0, layer.kv_stride):
                out[off + d * stride: off + d * stride + layer.segment_bytes] = \
                    fill[off + s * stride: off + s * stride + layer.segment_bytes]
        else:
            nb = layer.segment_bytes * layer.segments
            out[d * stride: d * stride + nb] = fill[s * stride: s * stride + nb]
    return out
