"""ctypes view of the C oracle (``pf_oracle.c``) plus the small pieces restated in Python.

TEST INFRASTRUCTURE ONLY: nothing in the product package imports this module.  It is the
checker for the CUDA path (tests, smoke check, the benchmark's CPU-baseline/reference legs).
"""

from __future__ import annotations

import ctypes as C
import os
import struct
import subprocess
from dataclasses import dataclass
from typing import Optional, Sequence

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libpf_oracle.so")
_ERRLEN = 512


def build(force: bool = False) -> str:
    """Compile ``pf_oracle.c`` with gcc (through the Makefile beside it)."""
    src_mtime = max(os.path.getmtime(os.path.join(_HERE, f)) for f in ("pf_oracle.c", "pf_oracle.h"))
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < src_mtime:
        subprocess.check_call(["make", "-s", "-C", _HERE, "-B", "libpf_oracle.so"])
    return _LIB_PATH


class Layout(C.Structure):
    _fields_ = [
        ("data_ptr", C.c_uint64),
        ("size_bytes", C.c_size_t),
        ("num_blocks", C.c_size_t),
        ("block_stride_bytes", C.c_size_t),
        ("segment_bytes", C.c_size_t),
        ("segments", C.c_size_t),
        ("padded_segment_bytes", C.c_size_t),
        ("split", C.c_int),
        ("kv_stride_bytes", C.c_size_t),
    ]


class CopyDesc(C.Structure):
    _fields_ = [
        ("device", C.c_uint64),
        ("host", C.c_uint64),
        ("host_device", C.c_uint64),
        ("size", C.c_size_t),
        ("device_allocation", C.c_size_t),
        ("host_allocation", C.c_size_t),
    ]

    def as_tuple(self):
        return (self.device, self.host, self.host_device, self.size, self.device_allocation, self.host_allocation)


class HostBlock(C.Structure):
    _fields_ = [
        ("block_idx", C.c_size_t),
        ("n_segments", C.c_size_t),
        ("seg_host", C.c_uint64 * 2),
        ("seg_host_device", C.c_uint64 * 2),
        ("seg_allocation", C.c_size_t * 2),
        ("host_offset", C.c_size_t),
    ]


class LayerTask(C.Structure):
    _fields_ = [("layout", Layout), ("n_blocks", C.c_size_t), ("blocks", C.POINTER(HostBlock))]


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        L.pfo_layout_new.argtypes = [C.POINTER(Layout), C.c_uint64, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t,
                                     C.c_size_t, C.c_char_p, C.c_size_t]
        L.pfo_layout_new.restype = C.c_int
        L.pfo_layout_with_block_stride.argtypes = [C.POINTER(Layout), C.c_size_t, C.c_char_p, C.c_size_t]
        L.pfo_layout_with_block_stride.restype = C.c_int
        L.pfo_layout_with_ssd_padding.argtypes = [C.POINTER(Layout), C.c_size_t]
        L.pfo_layout_with_ssd_padding.restype = None
        L.pfo_layout_padded_block_bytes.argtypes = [C.POINTER(Layout)]
        L.pfo_layout_padded_block_bytes.restype = C.c_size_t
        L.pfo_layout_block_copies.argtypes = [C.POINTER(Layout), C.c_size_t, C.POINTER(C.c_uint64),
                                              C.POINTER(C.c_size_t), C.c_char_p, C.c_size_t]
        L.pfo_layout_block_copies.restype = C.c_int
        L.pfo_build_page_layout.argtypes = [C.POINTER(C.c_size_t), C.POINTER(C.c_size_t), C.c_size_t, C.c_size_t,
                                            C.POINTER(C.c_size_t)] + [C.POINTER(C.c_size_t)] * 5 + [C.c_char_p,
                                                                                                   C.c_size_t]
        L.pfo_build_page_layout.restype = C.c_int
        L.pfo_build_copy_descs.argtypes = [C.POINTER(LayerTask), C.c_size_t, C.POINTER(CopyDesc), C.c_size_t,
                                           C.POINTER(C.c_size_t), C.c_char_p, C.c_size_t]
        L.pfo_build_copy_descs.restype = C.c_long
        L.pfo_merge.argtypes = [C.POINTER(CopyDesc), C.c_size_t, C.POINTER(CopyDesc)]
        L.pfo_merge.restype = C.c_size_t
        L.pfo_execute.argtypes = [C.POINTER(CopyDesc), C.c_size_t, C.c_int]
        L.pfo_execute.restype = None
        L.pfo_execute_mt.argtypes = [C.POINTER(CopyDesc), C.c_size_t, C.c_int, C.c_int]
        L.pfo_execute_mt.restype = C.c_double
        L.pfo_pool_unit_size.argtypes = [C.c_uint64, C.c_uint64]
        L.pfo_pool_unit_size.restype = C.c_uint64
        _lib = L
    return _lib


class OracleError(ValueError):
    """A validation failure reported by the oracle; the message is the reference's text."""


def _err():
    return C.create_string_buffer(_ERRLEN)


class KVCacheLayout:
    """Python handle on a ``pfo_layout`` (pegaflow-core/src/layout.rs:43-62)."""

    def __init__(self, data_ptr, size_bytes, num_blocks, segment_bytes, kv_stride_bytes, segments):
        self.c = Layout()
        e = _err()
        if lib().pfo_layout_new(C.byref(self.c), data_ptr, size_bytes, num_blocks, segment_bytes, kv_stride_bytes,
                                segments, e, _ERRLEN) != 0:
            raise OracleError(e.value.decode())

    def with_block_stride(self, stride) -> "KVCacheLayout":
        e = _err()
        if lib().pfo_layout_with_block_stride(C.byref(self.c), stride, e, _ERRLEN) != 0:
            raise OracleError(e.value.decode())
        return self

    def with_ssd_padding(self, alignment) -> "KVCacheLayout":
        lib().pfo_layout_with_ssd_padding(C.byref(self.c), alignment)
        return self

    def block_copies(self, block_idx):
        """[(addr, bytes)] — one entry for a contiguous block, two (K, V) for a split block."""
        addr = (C.c_uint64 * 2)()
        nbytes = (C.c_size_t * 2)()
        e = _err()
        n = lib().pfo_layout_block_copies(C.byref(self.c), block_idx, addr, nbytes, e, _ERRLEN)
        if n < 0:
            raise OracleError(e.value.decode())
        return [(addr[i], nbytes[i]) for i in range(n)]

    is_split = property(lambda self: bool(self.c.split))
    num_blocks = property(lambda self: self.c.num_blocks)
    segment_bytes = property(lambda self: self.c.segment_bytes)
    segments = property(lambda self: self.c.segments)
    padded_segment_bytes = property(lambda self: self.c.padded_segment_bytes)
    padded_block_bytes = property(lambda self: self.c.padded_segment_bytes * self.c.segments)
    block_bytes = property(lambda self: self.c.segment_bytes * self.c.segments)


def build_page_layout(worker_layer_sets: Sequence[Sequence[int]], n_layers: int, padded_bytes: Sequence[int]):
    """instance.rs:107-162.  Returns dict(layer_shard, layer_offsets, layer_bytes, shard_page_sizes)."""
    sets = [sorted(set(s)) for s in worker_layer_sets]
    offsets = [0]
    items = []
    for s in sets:
        items.extend(s)
        offsets.append(len(items))
    SZ = C.c_size_t
    c_off = (SZ * len(offsets))(*offsets)
    c_items = (SZ * max(1, len(items)))(*items)
    c_pad = (SZ * max(1, n_layers))(*padded_bytes)
    shard = (SZ * max(1, n_layers))()
    loff = (SZ * max(1, n_layers))()
    lbytes = (SZ * max(1, n_layers))()
    pages = (SZ * max(1, len(sets)))()
    n_shards = SZ()
    e = _err()
    rc = lib().pfo_build_page_layout(c_off, c_items, len(sets), n_layers, c_pad, shard, loff, lbytes, pages,
                                     C.byref(n_shards), e, _ERRLEN)
    if rc != 0:
        raise OracleError(e.value.decode())
    return {
        "layer_shard": list(shard[:n_layers]),
        "layer_offsets": list(loff[:n_layers]),
        "layer_bytes": list(lbytes[:n_layers]),
        "shard_page_sizes": list(pages[: n_shards.value]),
    }


@dataclass
class HostSeg:
    host: int
    host_device: int
    allocation: int


def build_copy_descs(layers):
    """gpu_worker.rs:353-423.  ``layers`` = [(KVCacheLayout, [(block_idx, [HostSeg...], host_offset)])].

    Returns (ctypes CopyDesc array, count, total_bytes)."""
    tasks = (LayerTask * max(1, len(layers)))()
    keep = []
    cap = 0
    for li, (layout, blocks) in enumerate(layers):
        arr = (HostBlock * max(1, len(blocks)))()
        for bi, (block_idx, segs, host_offset) in enumerate(blocks):
            hb = arr[bi]
            hb.block_idx = block_idx
            hb.n_segments = len(segs)
            for si, s in enumerate(segs[:2]):
                hb.seg_host[si] = s.host
                hb.seg_host_device[si] = s.host_device
                hb.seg_allocation[si] = s.allocation
            hb.host_offset = host_offset
        keep.append(arr)
        tasks[li].layout = layout.c
        tasks[li].n_blocks = len(blocks)
        tasks[li].blocks = arr
        cap += 2 * len(blocks)
    out = (CopyDesc * max(1, cap))()
    total = C.c_size_t()
    e = _err()
    n = lib().pfo_build_copy_descs(tasks, len(layers), out, cap, C.byref(total), e, _ERRLEN)
    if n < 0:
        raise OracleError(e.value.decode())
    return out, n, total.value


def merge(descs, n):
    """transfer/memcpy.rs:25-55."""
    out = (CopyDesc * max(1, n))()
    m = lib().pfo_merge(descs, n, out)
    return out, m


def execute(descs, n, host_is_src: bool, threads: int = 1) -> float:
    """Run the batch with memcpy semantics; returns elapsed seconds."""
    return lib().pfo_execute_mt(descs, n, 1 if host_is_src else 0, threads)


def pool_unit_size(pool_size: int, hint: Optional[int] = None) -> int:
    return lib().pfo_pool_unit_size(pool_size, hint or 0)


# ----------------------------------------------------------------------------------------------
# Small pieces restated directly in Python.
# ----------------------------------------------------------------------------------------------

def group_hash(h: bytes, group_id: int) -> bytes:
    """pegaflow-common/src/block.rs:35-43: group 0 keeps the raw hash; others append the
    big-endian group id."""
    if group_id == 0:
        return bytes(h)
    return bytes(h) + struct.pack(">I", group_id)


LOAD_STATE_MAGIC = 0x50464C44
LOAD_STATE_VERSION = 1
LOAD_STATE_PENDING, LOAD_STATE_SUCCESS, LOAD_STATE_ERROR = 0, 1, -1
LOAD_STATE_SHM_BYTES = 8 + 16 + 8


def load_state_image(state: int = LOAD_STATE_PENDING) -> bytes:
    """Bytes of a freshly created LoadState mapping (pegaflow-core/src/sync_state.rs:23-47,
    190-249): an 8-byte offset word (8 for a page-aligned mapping), then at that offset
    {u32 magic, u32 version, i64 state}; the mapping is 32 bytes long."""
    return struct.pack("<QIIq", 8, LOAD_STATE_MAGIC, LOAD_STATE_VERSION, state) + b"\0" * 8


def parse_load_state(buf: bytes) -> int:
    """Attach-side validation of sync_state.rs:251-302; returns the state or raises."""
    if len(buf) < LOAD_STATE_SHM_BYTES:
        raise OracleError(f"shared memory too small (actual={len(buf)} bytes, required={LOAD_STATE_SHM_BYTES} bytes)")
    (offset,) = struct.unpack_from("<Q", buf, 0)
    if offset < 8:
        raise OracleError(f"invalid LoadState offset (offset={offset}, len={len(buf)}) recorded in shared memory")
    if offset + 16 > len(buf):
        raise OracleError(f"shared memory too small (actual={len(buf)} bytes, required={offset + 16} bytes)")
    if offset % 8:
        raise OracleError("misaligned LoadState")
    magic, version, state = struct.unpack_from("<IIq", buf, offset)
    if magic != LOAD_STATE_MAGIC or version != LOAD_STATE_VERSION:
        raise OracleError(f"invalid LoadState header (magic={magic:#x}, version={version}, "
                          f"expected magic={LOAD_STATE_MAGIC:#x}, version={LOAD_STATE_VERSION})")
    return state


def infer_kv_cache_registration(shape, stride, element_size, logical_block_size, *, is_mla=False,
                                is_recurrent_state=False):
    """python/pegaflow/connector/worker.py:65-151 restated on plain tuples.

    Returns dict(layout, num_blocks, bytes_per_block, kv_stride_bytes, segments,
    physical_blocks_per_logical_block)."""
    shape, stride = tuple(shape), tuple(stride)
    if logical_block_size <= 0:
        raise ValueError(f"logical block size must be > 0, got {logical_block_size}")
    if is_recurrent_state or not is_mla:
        if not is_recurrent_state and len(shape) >= 2 and shape[0] == 2:
            out = dict(layout="KV-first", num_blocks=shape[1], bytes_per_block=stride[1] * element_size,
                       kv_stride_bytes=stride[0] * element_size, segments=2)
        else:
            out = dict(layout="blocks-first", num_blocks=shape[0], bytes_per_block=stride[0] * element_size,
                       kv_stride_bytes=0, segments=1)
        if out["num_blocks"] <= 0:
            raise ValueError(f"physical block count must be > 0, got {out['num_blocks']}")
        if out["bytes_per_block"] == 0:
            raise ValueError(f"Invalid bytes_per_block: shape={shape} stride={stride}")
        out["physical_blocks_per_logical_block"] = 1
        return out
    phys_blocks = shape[0]
    phys_block_size = shape[1] if len(shape) >= 2 else logical_block_size
    phys_bytes = stride[0] * element_size
    if phys_blocks <= 0:
        raise ValueError(f"physical block count must be > 0, got {phys_blocks}")
    if phys_block_size <= 0:
        raise ValueError(f"physical block size must be > 0, got {phys_block_size}")
    if logical_block_size % phys_block_size != 0:
        raise ValueError("logical block size must be a multiple of physical block size "
                         f"(logical={logical_block_size}, physical={phys_block_size})")
    ratio = logical_block_size // phys_block_size
    if phys_blocks % ratio != 0:
        raise ValueError("physical block count must be divisible by physical/logical split ratio "
                         f"(physical_blocks={phys_blocks}, ratio={ratio})")
    bpb = phys_bytes * ratio
    if bpb == 0:
        raise ValueError(f"Invalid bytes_per_block: shape={shape} stride={stride}")
    return dict(layout="blocks-first", num_blocks=phys_blocks // ratio, bytes_per_block=bpb, kv_stride_bytes=0,
                segments=1, physical_blocks_per_logical_block=ratio)
