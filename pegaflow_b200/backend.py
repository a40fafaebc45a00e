"""Python view of the backend boundary: batches of copies enqueued on a CUDA stream.

Mirrors ``trait TransferBackend`` of the reference (pegaflow-core/src/transfer/mod.rs:53-60)
plus the descriptor-free layer form and the NVLink peer copy.  Streams and events are passed
as integer handles (``torch.cuda.Stream.cuda_stream`` / ``torch.cuda.Event.cuda_event``).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

from . import _native as N


def _release(fn_name, handle, _release_native=N.release):
    # bound at definition time: a finalizer may run after module globals were cleared
    _release_native(fn_name, handle)


@dataclass
class HostRun:
    first_block: int
    n_blocks: int
    host: int
    host_device: int
    stride_bytes: int


@dataclass
class LayerXfer:
    """One layer of a save/load: affine device layout, block ids, host runs per device range."""
    data_ptr: int
    block_stride_bytes: int
    kv_stride_bytes: int
    range_bytes: int
    n_ranges: int
    block_ids: Sequence[int]
    runs: List[List[HostRun]] = field(default_factory=list)


class PinnedPool:
    """`PinnedAllocator` of the reference (pinned_pool.rs:616-715) through the C ABI."""

    def __init__(self, nbytes: int, *, use_hugepages=False, use_mmap=False, numa_node=-1, unit_hint=0, shards=1,
                 transparent_huge=False):
        cfg = N.PoolConfig(int(use_hugepages), int(use_mmap or transparent_huge), numa_node, unit_hint, shards,
                           int(transparent_huge))
        h = C.c_void_p()
        N.check(N.lib.pf_pool_new(nbytes, C.byref(cfg), C.byref(h)))
        self._h = h

    def close(self):
        if getattr(self, "_h", None):
            _release("pf_pool_free", self._h)
            self._h = None

    __del__ = close

    def alloc(self, nbytes: int):
        """Returns (host_address, device_address, handle)."""
        host, dev, handle = C.c_void_p(), C.c_uint64(), C.c_uint64()
        N.check(N.lib.pf_pool_alloc(self._h, nbytes, C.byref(host), C.byref(dev), C.byref(handle)))
        return host.value, dev.value, handle.value

    def release(self, handle: int):
        N.check(N.lib.pf_pool_release(self._h, handle))

    def usage(self):
        used, total, largest = C.c_uint64(), C.c_uint64(), C.c_uint64()
        N.check(N.lib.pf_pool_usage(self._h, C.byref(used), C.byref(total), C.byref(largest)))
        return used.value, total.value, largest.value


class TransferBackend:
    def __init__(self, device_id: int = 0, *, route: int = N.ROUTE_AUTO, staging_slot_bytes: int = 0,
                 staging_slots: int = 0, pack_ctas: int = 0, link_ctas: int = 0, min_dma_bytes: int = 0,
                 time_kernels: bool = False, copy_streams: int = 0, gather_slots: int = 0):
        cfg = N.BackendConfig(staging_slot_bytes, staging_slots, pack_ctas, link_ctas, min_dma_bytes, route,
                              int(time_kernels), copy_streams, gather_slots)
        h = C.c_void_p()
        N.check(N.lib.pf_backend_new(device_id, C.byref(cfg), C.byref(h)))
        self._h = h

    def close(self):
        if getattr(self, "_h", None):
            _release("pf_backend_free", self._h)
            self._h = None

    __del__ = close

    def name(self) -> str:
        return N.lib.pf_backend_name(self._h).decode()

    @staticmethod
    def make_descs(copies):
        """copies: iterable of (device, host, host_device, size[, device_allocation, host_allocation])."""
        copies = list(copies)
        arr = (N.CopyDesc * max(1, len(copies)))()
        for i, c in enumerate(copies):
            arr[i].device, arr[i].host, arr[i].host_device, arr[i].size = c[0], c[1], c[2], c[3]
            arr[i].device_allocation = c[4] if len(c) > 4 else 0
            arr[i].host_allocation = c[5] if len(c) > 5 else 0
        return arr, len(copies)

    def h2d(self, descs, n: int, stream: int = 0):
        N.check(N.lib.pf_backend_h2d(self._h, descs, n, C.c_void_p(stream or None)))

    def d2h(self, descs, n: int, stream: int = 0):
        N.check(N.lib.pf_backend_d2h(self._h, descs, n, C.c_void_p(stream or None)))

    @staticmethod
    def make_layers(layers: Sequence[LayerXfer]):
        arr = (N.LayerXfer * max(1, len(layers)))()
        keep = []
        for i, L in enumerate(layers):
            import numpy as np

            ids_np = np.ascontiguousarray(L.block_ids, dtype=np.uint32)
            ids = ids_np.ctypes.data_as(C.POINTER(C.c_uint32))
            keep.append(ids_np)
            a = arr[i]
            a.data_ptr, a.block_stride_bytes, a.kv_stride_bytes = L.data_ptr, L.block_stride_bytes, L.kv_stride_bytes
            a.range_bytes, a.n_ranges, a.n_blocks = L.range_bytes, L.n_ranges, len(L.block_ids)
            a.block_ids = ids
            for r in range(2):
                runs = L.runs[r] if r < len(L.runs) else []
                ra = (N.HostRun * max(1, len(runs)))()
                for j, run in enumerate(runs):
                    ra[j] = N.HostRun(run.first_block, run.n_blocks, run.host, run.host_device, run.stride_bytes)
                keep.append(ra)
                a.n_runs[r] = len(runs)
                a.runs[r] = ra
        return arr, len(layers), keep

    def _events(self, layer_done, n):
        if layer_done is None:
            return None
        return (C.c_void_p * max(1, n))(*[C.c_void_p(e or None) for e in layer_done])

    def save_layers(self, layers, stream: int = 0, layer_done: Optional[Sequence[int]] = None):
        arr, n, keep = layers if isinstance(layers, tuple) else self.make_layers(layers)
        N.check(N.lib.pf_backend_save_layers(self._h, arr, n, C.c_void_p(stream or None), self._events(layer_done, n)))

    def load_layers(self, layers, stream: int = 0, layer_done: Optional[Sequence[int]] = None):
        arr, n, keep = layers if isinstance(layers, tuple) else self.make_layers(layers)
        N.check(N.lib.pf_backend_load_layers(self._h, arr, n, C.c_void_p(stream or None), self._events(layer_done, n)))

    def gather_layers(self, layers, stream: int = 0):
        """The gather kernels of a staged save without the DMA (nothing reaches the host): for timing
        the kernel alone.  Synchronise the stream before the next real transfer on this backend."""
        arr, n, keep = layers if isinstance(layers, tuple) else self.make_layers(layers)
        N.check(N.lib.pf_backend_gather_layers(self._h, arr, n, C.c_void_p(stream or None)))

    def peer_copy(self, src_layout, src_ids, dst_layout, dst_ids, stream: int = 0):
        """layouts: (data_ptr, block_stride_bytes, kv_stride_bytes, range_bytes, n_ranges[, num_blocks])."""
        import numpy as np

        n = len(src_ids)
        if len(dst_ids) != n:
            raise N.PegaflowInvalidArgument(3, "invalid argument: peer copy needs one destination per source block")
        sa = np.ascontiguousarray(src_ids, dtype=np.uint32)
        da = np.ascontiguousarray(dst_ids, dtype=np.uint32)
        s, d = N.DeviceLayout(*src_layout), N.DeviceLayout(*dst_layout)
        U = C.POINTER(C.c_uint32)
        N.check(N.lib.pf_backend_peer_copy(self._h, C.byref(s), sa.ctypes.data_as(U), C.byref(d), da.ctypes.data_as(U), n,
                                           C.c_void_p(stream or None)))

    def peer_copy_layers(self, src_layouts, src_ids, dst_layouts, dst_ids, stream: int = 0):
        """One call for every layer of a prefix hit: the layers share the block ids."""
        import numpy as np

        n = len(src_ids)
        if len(dst_ids) != n:
            raise N.PegaflowInvalidArgument(3, "invalid argument: peer copy needs one destination per source block")
        if len(src_layouts) != len(dst_layouts):
            raise N.PegaflowInvalidArgument(3, "invalid argument: peer copy needs one destination layout per source layout")
        sa = np.ascontiguousarray(src_ids, dtype=np.uint32)
        da = np.ascontiguousarray(dst_ids, dtype=np.uint32)
        L = len(src_layouts)
        s = (N.DeviceLayout * L)(*[N.DeviceLayout(*x) for x in src_layouts])
        d = (N.DeviceLayout * L)(*[N.DeviceLayout(*x) for x in dst_layouts])
        U = C.POINTER(C.c_uint32)
        N.check(N.lib.pf_backend_peer_copy_layers(self._h, s, d, L, sa.ctypes.data_as(U), da.ctypes.data_as(U), n,
                                                  C.c_void_p(stream or None)))

    def stats(self) -> dict:
        st = N.BackendStats()
        N.check(N.lib.pf_backend_get_stats(self._h, C.byref(st)))
        return {f: getattr(st, f) for f, _ in N.BackendStats._fields_}


def numa_node_of_device(device_id: int) -> int:
    """NUMA node of a CUDA device from sysfs, -1 when unknown (pegaflow-common/src/numa.rs:344-411)."""
    return int(N.lib.pf_numa_node_of_device(device_id))


def enable_peer_access(device_id: int, peer_device: int):
    N.check(N.lib.pf_enable_peer_access(device_id, peer_device))


def save_blocks_noalloc(device_id: int, layout, block_ids, host_dst: int, host_dst_bytes: int, stream: int = 0):
    """Allocation-free save of a small batch (``pf_save_blocks_noalloc``).

    For callers that must not allocate device memory at that moment (no free HBM left, no
    tolerance for cudaMalloc's device-wide synchronisation, a stream capture in progress).  The
    staging area lives inside the library image; at most ``NOALLOC_MAX_BLOCKS`` blocks and
    ``NOALLOC_MAX_PAYLOAD_BYTES`` bytes per call.  ``layout`` is (data_ptr, block_stride_bytes,
    kv_stride_bytes, range_bytes, n_ranges[, num_blocks]); with ``num_blocks`` given, ids outside
    the cache are rejected before anything is launched.  ``host_dst`` should be page-locked.  Calls
    on one device share the staging area: do not let their GPU work overlap.  Make the first call
    on a device (an empty batch will do) before any stream capture."""
    n = len(block_ids)
    ids = (C.c_uint32 * max(1, n))(*[int(b) for b in block_ids])
    lay = N.DeviceLayout(*layout)
    N.check(N.lib.pf_save_blocks_noalloc(device_id, C.byref(lay), ids, n, C.c_void_p(host_dst), host_dst_bytes,
                                         C.c_void_p(stream or None)))
