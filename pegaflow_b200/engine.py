"""Python view of the engine boundary of ``libpegaflow_b200.so``.

``PegaEngine`` carries the reference's method names and argument order
(pegaflow-core/src/lib.rs:138-709, offload.rs:293-300) so that code written against the
reference's engine reads the same.  Every call goes through the C ABI; nothing here moves
bytes on the CPU.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import numpy as np

from . import _native as N
from ._native import PegaFlowError, PegaflowInternal, PegaflowInvalidArgument  # noqa: F401  (re-exported)

def _release(fn_name, handle, _release_native=N.release):
    # bound at definition time: a finalizer may run after module globals were cleared
    _release_native(fn_name, handle)


TRANSFER_MODES = {"direct": 0, "kernel": 1}  # transfer/mod.rs:66-76; both run on the one B200 backend

LOAD_STATE_PENDING, LOAD_STATE_SUCCESS, LOAD_STATE_ERROR = 0, 1, -1


def _hash_arrays(hashes: Sequence[bytes]):
    """(keep-alive, pointer array, length array) for a list of hashes: one contiguous copy of the bytes
    and two numpy arrays, not one ctypes object per hash (a 10 K-token prompt has 640 of them per call)."""
    n = len(hashes)
    lens = np.fromiter((len(h) for h in hashes), dtype=np.uint64, count=n) if n else np.zeros(1, dtype=np.uint64)
    blob = np.frombuffer(b"".join(bytes(h) for h in hashes) + b"\0", dtype=np.uint8)
    ptrs = np.full(max(1, n), blob.ctypes.data, dtype=np.uint64)
    if n > 1:
        ptrs[1:] += np.cumsum(lens[:-1], dtype=np.uint64)
    return (blob, ptrs, lens), ptrs.ctypes.data_as(C.POINTER(C.POINTER(C.c_uint8))), lens.ctypes.data_as(C.POINTER(C.c_size_t))


class Block:
    """Handle on a sealed block (``Arc<SealedBlock>`` in the reference): owned, or a view of one entry
    of a BlockList, which then stays alive as long as the view does."""

    def __init__(self, handle, parent=None):
        self._h = handle
        self._parent = parent

    def __del__(self):
        if getattr(self, "_h", None) and getattr(self, "_parent", None) is None:
            _release("pf_block_release", self._h)
        self._h = None

    @property
    def num_slots(self) -> int:
        return N.lib.pf_block_num_slots(self._h)

    def slot_image(self, slot: int) -> List[bytes]:
        """Host bytes of one slot, one ``bytes`` per segment."""
        nseg = C.c_size_t()
        sizes = (C.c_size_t * 2)()
        N.check(N.lib.pf_block_slot_info(self._h, slot, C.byref(nseg), sizes))
        out = []
        for s in range(nseg.value):
            buf = C.create_string_buffer(sizes[s])
            N.check(N.lib.pf_block_slot_read(self._h, slot, s, buf, sizes[s]))
            out.append(buf.raw)
        return out


class BlockList:
    """The blocks a prefix query hit, as the one array of handles the C ABI filled: sequence of Block
    views, released in a single call.  A query for a 10 K-token prompt returns 640 handles; one Python
    object and two library calls per handle would cost more than the query itself."""

    def __init__(self, array, n):
        self._arr, self._n = array, n

    def __del__(self):
        if getattr(self, "_arr", None) is not None and self._n:
            _release_many(self._arr, self._n)
        self._arr = None

    def __len__(self):
        return self._n

    def __getitem__(self, i):
        if isinstance(i, slice):
            return [self[j] for j in range(*i.indices(self._n))]
        if i < 0:
            i += self._n
        if not 0 <= i < self._n:
            raise IndexError(i)
        return Block(C.c_void_p(self._arr[i]), parent=self)

    def __iter__(self):
        return (self[i] for i in range(self._n))

    def __eq__(self, other):
        return isinstance(other, (list, tuple, BlockList)) and len(other) == self._n and all(
            a is b or getattr(a, "_h", None) == getattr(b, "_h", 0) for a, b in zip(self, other))

    __hash__ = None


def _release_many(array, n, _module_dict=N.__dict__):
    # bound at definition time: a finalizer may run after module globals were cleared
    library = _module_dict.get("lib")
    if library is not None:
        library.pf_blocks_release(array, n)


class Completion:
    """Completion of an in-process load (the oneshot receiver of lib.rs:691-709)."""

    def __init__(self, handle):
        self._h = handle

    def __del__(self):
        if getattr(self, "_h", None):
            _release("pf_completion_free", self._h)
            self._h = None

    def poll(self) -> int:
        st = C.c_int()
        N.check(N.lib.pf_completion_poll(self._h, C.byref(st)))
        return st.value

    def wait(self, timeout: float = 120.0) -> int:
        st = C.c_int()
        N.check(N.lib.pf_completion_wait(self._h, timeout, C.byref(st)))
        return st.value

    def error(self) -> str:
        return N.lib.pf_completion_error(self._h).decode(errors="replace")


class PyLoadState:
    """Shared-memory load state (python/src/lib.rs:628-663 `PyLoadState`)."""

    def __init__(self, attach_to: Optional[str] = None):
        h = C.c_void_p()
        if attach_to is None:
            N.check(N.lib.pf_load_state_new(C.byref(h)))
        else:
            N.check(N.lib.pf_load_state_attach(attach_to.encode(), C.byref(h)))
        self._h = h

    def __del__(self):
        if getattr(self, "_h", None):
            _release("pf_load_state_free", self._h)
            self._h = None

    def shm_name(self) -> str:
        return N.lib.pf_load_state_shm_name(self._h).decode()

    def get_state(self) -> int:
        return N.lib.pf_load_state_get(self._h)

    def is_ready(self) -> bool:
        return self.get_state() != LOAD_STATE_PENDING

    def set_completed(self):
        N.lib.pf_load_state_set_completed(self._h)

    def set_error(self):
        N.lib.pf_load_state_set_error(self._h)


class PegaEngine:
    def __init__(self, pool_bytes: int, use_hugepages: bool = False, *, enable_numa_affinity: bool = True,
                 blockwise_alloc: bool = False, hint_value_size: int = 0, pool_shards: int = 1,
                 host_alignment: int = 0, use_mmap_pool: bool = False, route: int = N.ROUTE_AUTO,
                 staging_slot_bytes: int = 0, staging_slots: int = 0, min_dma_bytes: int = 0, link_ctas: int = 0,
                 pack_ctas: int = 0, time_kernels: bool = False, copy_streams: int = 0, gather_slots: int = 0):
        cfg = N.StorageConfig()
        cfg.enable_numa_affinity = int(enable_numa_affinity)
        cfg.blockwise_alloc = int(blockwise_alloc)
        cfg.hint_value_size = hint_value_size
        cfg.pool_shards = pool_shards
        cfg.host_alignment = host_alignment
        cfg.use_mmap_pool = int(use_mmap_pool)
        cfg.backend.route = route
        cfg.backend.staging_slot_bytes = staging_slot_bytes
        cfg.backend.staging_slots = staging_slots
        cfg.backend.min_dma_bytes = min_dma_bytes
        cfg.backend.link_ctas = link_ctas
        cfg.backend.pack_ctas = pack_ctas
        cfg.backend.time_kernels = int(time_kernels)
        cfg.backend.copy_streams = copy_streams
        cfg.backend.gather_slots = gather_slots
        h = C.c_void_p()
        N.check(N.lib.pf_engine_new(pool_bytes, int(use_hugepages), C.byref(cfg), C.byref(h)))
        self._h = h

    def close(self):
        if getattr(self, "_h", None):
            _release("pf_engine_free", self._h)
            self._h = None

    __del__ = close

    # lib.rs:302-322
    def register_context_layer_batch_strided(self, instance_id, namespace, device_id, tp_rank, pp_rank, tp_size,
                                             world_size, layer_names, data_ptrs, size_bytes, num_blocks,
                                             bytes_per_block, kv_stride_bytes, segments, block_stride_bytes=None,
                                             layer_group_ids=None, transfer_mode="direct", page_first=False):
        n = len(layer_names)
        lists = dict(data_ptrs=data_ptrs, size_bytes=size_bytes, num_blocks=num_blocks, bytes_per_block=bytes_per_block,
                     kv_stride_bytes=kv_stride_bytes, segments=segments)
        if any(len(v) != n for v in lists.values()):
            # lib.rs:327-344: the C ABI takes one length, so the mismatch is caught here
            raise PegaflowInvalidArgument(3, "invalid argument: registration metadata length mismatch: layer_names="
                                          f"{n}, " + ", ".join(f"{k}={len(v)}" for k, v in lists.items()))
        for key, v in (("block_stride_bytes", block_stride_bytes), ("layer_group_ids", layer_group_ids)):
            if v is not None and len(v) != n:
                raise PegaflowInvalidArgument(3, "invalid argument: registration metadata length mismatch: "
                                              f"layer_names={n}, {key}={len(v)}")
        SZ = C.c_size_t * max(1, n)
        names = (C.c_char_p * max(1, n))(*[s.encode() for s in layer_names])
        mode = TRANSFER_MODES[transfer_mode] if isinstance(transfer_mode, str) else int(transfer_mode)
        N.check(N.lib.pf_engine_register_context_layer_batch_strided(
            self._h, instance_id.encode(), namespace.encode(), device_id, tp_rank, pp_rank, tp_size, world_size, n,
            names, (C.c_uint64 * max(1, n))(*data_ptrs), SZ(*size_bytes), SZ(*num_blocks), SZ(*bytes_per_block),
            SZ(*kv_stride_bytes), SZ(*segments), SZ(*block_stride_bytes) if block_stride_bytes is not None else None,
            (C.c_uint32 * max(1, n))(*layer_group_ids) if layer_group_ids is not None else None, mode,
            int(bool(page_first))))

    def unregister_instance(self, instance_id):
        N.check(N.lib.pf_engine_unregister_instance(self._h, instance_id.encode()))

    def list_instance_ids(self):
        """lib.rs:477-484; sorted."""
        buf, need = C.create_string_buffer(1 << 16), N.sz()
        N.check(N.lib.pf_engine_list_instances(self._h, buf, len(buf), C.byref(need)))
        if need.value > len(buf):
            buf = C.create_string_buffer(need.value)
            N.check(N.lib.pf_engine_list_instances(self._h, buf, len(buf), C.byref(need)))
        return [s for s in buf.value.decode().split("\n") if s]

    def unregister_all_instances(self):
        """lib.rs:459-475: removes every instance (their leases go with them) and returns the ids."""
        buf, need = C.create_string_buffer(1 << 20), N.sz()
        N.check(N.lib.pf_engine_unregister_all_instances(self._h, buf, len(buf), C.byref(need)))
        return [s for s in buf.value.decode().split("\n") if s]

    def instance_namespace(self, instance_id):
        """lib.rs:487-489."""
        buf, need = C.create_string_buffer(4096), N.sz()
        N.check(N.lib.pf_engine_instance_namespace(self._h, instance_id.encode(), buf, len(buf), C.byref(need)))
        return buf.value.decode()

    def _layer_saves(self, saves):
        n = len(saves)
        arr = (N.LayerSave * max(1, n))()
        keep = []
        marshalled, marshalled_ids = {}, {}   # layers usually share one hash list and one id list: marshal once
        for i, (name, ids, hashes) in enumerate(saves):
            if len(ids) != len(hashes):
                raise PegaflowInvalidArgument(3, f"invalid argument: block_ids length {len(ids)} does not match "
                                              f"block_hashes {len(hashes)} for layer {name}")
            if id(hashes) not in marshalled:
                marshalled[id(hashes)] = _hash_arrays(hashes)
            bufs, ptrs, lens = marshalled[id(hashes)]
            if id(ids) not in marshalled_ids:
                a = np.ascontiguousarray(ids, dtype=np.uint64) if len(ids) else np.zeros(1, dtype=np.uint64)
                marshalled_ids[id(ids)] = (a, a.ctypes.data_as(C.POINTER(C.c_size_t)))
            ids_np, ids_arr = marshalled_ids[id(ids)]
            keep.append((bufs, ptrs, lens, ids_np, ids_arr))
            arr[i].layer_name = name.encode()
            arr[i].n_blocks = len(ids)
            arr[i].block_ids = ids_arr
            arr[i].block_hashes = ptrs
            arr[i].block_hash_lens = lens
        return arr, n, keep

    # offload.rs:293-300
    def prepare_saves(self, saves):
        """Marshal `saves` once; the result can be passed to batch_save / save_layers_async
        repeatedly (what a native caller of the C ABI would hold anyway)."""
        return self._layer_saves(saves)

    def batch_save(self, instance_id, tp_rank, pp_rank, device_id, saves):
        """saves: [(layer_name, block_ids, block_hashes)] or the result of prepare_saves()."""
        arr, n, _keep = saves if isinstance(saves, tuple) else self._layer_saves(saves)
        N.check(N.lib.pf_engine_batch_save(self._h, instance_id.encode(), tp_rank, pp_rank, device_id, n, arr))

    def save_layers_async(self, instance_id, tp_rank, pp_rank, device_id, saves, ready_event: int = 0):
        """Non-blocking save that starts once ``ready_event`` (a cudaEvent_t value or 0) fired."""
        arr, n, _keep = saves if isinstance(saves, tuple) else self._layer_saves(saves)
        N.check(N.lib.pf_engine_save_layers_async(self._h, instance_id.encode(), tp_rank, pp_rank, device_id, n, arr,
                                                  C.c_void_p(ready_event or None)))

    def flush_saves(self):
        N.check(N.lib.pf_engine_flush_saves(self._h))

    # lib.rs:506-533
    @staticmethod
    def prepare_hashes(hashes: Sequence[bytes]):
        return ("hashes", len(hashes)) + _hash_arrays(hashes)

    def query_prefix(self, instance_id, hashes, req_id: str = ""):
        if isinstance(hashes, tuple) and hashes and hashes[0] == "hashes":
            _tag, n, _bufs, ptrs, lens = hashes
        else:
            n = len(hashes)
            _bufs, ptrs, lens = _hash_arrays(hashes)
        out = (C.c_void_p * max(1, n))()
        hit, missing = C.c_size_t(), C.c_size_t()
        N.check(N.lib.pf_engine_query_prefix(self._h, instance_id.encode(), req_id.encode(), n, ptrs, lens, out,
                                             C.byref(hit), C.byref(missing)))
        return BlockList(out, hit.value), missing.value

    def query_group_membership(self, instance_id, group_id, hashes: Sequence[bytes]):
        n = len(hashes)
        _bufs, ptrs, lens = _hash_arrays(hashes)
        out = (C.c_void_p * max(1, n))()
        N.check(N.lib.pf_engine_query_group_membership(self._h, instance_id.encode(), group_id, n, ptrs, lens, out))
        return [Block(C.c_void_p(out[i])) if out[i] else None for i in range(n)]

    def create_query_lease(self, instance_id, blocks) -> bytes:
        n = len(blocks)
        arr = blocks._arr if isinstance(blocks, BlockList) else (C.c_void_p * max(1, n))(*[b._h for b in blocks])
        lease = (C.c_uint8 * 16)()
        N.check(N.lib.pf_engine_create_query_lease(self._h, instance_id.encode(), n, arr, lease))
        return bytes(lease)

    def release_query_lease(self, lease: bytes) -> bool:
        released = C.c_int()
        N.check(N.lib.pf_engine_release_query_lease(self._h, (C.c_uint8 * 16)(*lease), C.byref(released)))
        return bool(released.value)

    def _load_args(self, layer_groups, loads):
        flat = [nm.encode() for g in layer_groups for nm in g]
        groups = N.LayerGroups()
        groups.n_groups = len(layer_groups)
        sizes = (C.c_size_t * max(1, len(layer_groups)))(*[len(g) for g in layer_groups])
        names = (C.c_char_p * max(1, len(flat)))(*flat)
        groups.group_sizes = sizes
        groups.layer_names = names
        arr = (N.LeaseLoad * max(1, len(loads)))()
        keep = [sizes, names]
        for i, (lease, ids_by_group) in enumerate(loads):
            if len(ids_by_group) != len(layer_groups):
                raise PegaflowInvalidArgument(3, f"invalid argument: load group count {len(ids_by_group)} does not "
                                              f"match layer group count {len(layer_groups)}")
            n_blocks = len(ids_by_group[0]) if ids_by_group else 0
            for gi, g in enumerate(ids_by_group):
                if len(g) != n_blocks:
                    raise PegaflowInvalidArgument(3, "invalid argument: query lease destination lists differ in length "
                                                  f"({n_blocks} vs {len(g)} for group {gi})")
            rows = [(C.c_size_t * max(1, n_blocks))(*[N.PF_NO_BLOCK if v is None else int(v) for v in g])
                    for g in ids_by_group]
            ptrs = (C.POINTER(C.c_size_t) * max(1, len(rows)))(*[C.cast(r, C.POINTER(C.c_size_t)) for r in rows])
            keep.extend([rows, ptrs])
            arr[i].lease = (C.c_uint8 * 16)(*lease)
            arr[i].n_blocks = n_blocks
            arr[i].dst_ids = ptrs
        return groups, arr, len(loads), keep

    # lib.rs:691-709
    def prepare_loads(self, layer_groups, loads):
        return ("loads",) + self._load_args(layer_groups, loads)

    def batch_load_async(self, instance_id, tp_rank, device_id, layer_groups, loads=None) -> Completion:
        """`layer_groups` may be the result of prepare_loads(), in which case `loads` is unused."""
        if isinstance(layer_groups, tuple) and layer_groups and layer_groups[0] == "loads":
            _tag, groups, arr, n, _keep = layer_groups
        else:
            groups, arr, n, _keep = self._load_args(layer_groups, loads)
        out = C.c_void_p()
        N.check(N.lib.pf_engine_batch_load_inproc(self._h, instance_id.encode(), tp_rank, device_id, C.byref(groups),
                                                  n, arr, C.byref(out)))
        return Completion(out)

    def batch_load(self, instance_id, tp_rank, device_id, layer_groups, loads=None, timeout: float = 120.0):
        """Blocking convenience over batch_load_async: raises if the load fails."""
        done = self.batch_load_async(instance_id, tp_rank, device_id, layer_groups, loads)
        state = done.wait(timeout)
        if state == 0:
            raise PegaflowInternal(5, "storage error: load timed out")
        if state < 0:
            raise PegaflowInternal(5, done.error())

    # lib.rs:654-680
    def batch_load_shm(self, instance_id, tp_rank, device_id, load_state_shm: str, layer_groups, loads):
        groups, arr, n, _keep = self._load_args(layer_groups, loads)
        N.check(N.lib.pf_engine_batch_load_shm(self._h, instance_id.encode(), tp_rank, device_id,
                                               load_state_shm.encode(), C.byref(groups), n, arr))

    def layer_load_event(self, instance_id, device_id, layer_name) -> int:
        out = C.c_void_p()
        N.check(N.lib.pf_engine_layer_load_event(self._h, instance_id.encode(), device_id, layer_name.encode(),
                                                 C.byref(out)))
        return out.value or 0

    @staticmethod
    def stream_wait_event(stream: int, event: int):
        """Order `stream` (a cudaStream_t value, 0 = default stream) after `event`."""
        N.check(N.lib.pf_stream_wait_event(C.c_void_p(stream or None), C.c_void_p(event)))

    def peer_load(self, src_instance, src_device, dst_instance, dst_device, src_block_ids, dst_block_ids):
        n = len(src_block_ids)
        if len(dst_block_ids) != n:
            raise PegaflowInvalidArgument(3, "invalid argument: peer load needs one destination per source block")
        SZ = C.c_size_t * max(1, n)
        N.check(N.lib.pf_engine_peer_load(self._h, src_instance.encode(), src_device, dst_instance.encode(), dst_device,
                                          n, SZ(*src_block_ids), SZ(*dst_block_ids)))

    def metrics(self) -> dict:
        m = N.EngineMetrics()
        N.check(N.lib.pf_engine_get_metrics(self._h, C.byref(m)))
        out = {f: getattr(m, f) for f, _ in N.EngineMetrics._fields_ if f != "transfer"}
        out["transfer"] = {f: getattr(m.transfer, f) for f, _ in N.BackendStats._fields_}
        return out

    def cleanup_memory_cache(self) -> dict:
        """Drop every resident block from the cache (lib.rs:636-639): evicted_blocks, evicted_bytes,
        reclaimed_bytes (what the pool got back at once) and still_referenced_blocks (held by a lease, a
        load in flight or a caller's handle: their memory follows when the holder lets go)."""
        s = N.CacheCleanupStats()
        N.check(N.lib.pf_engine_cleanup_memory_cache(self._h, C.byref(s)))
        return {f: int(getattr(s, f)) for f, _ in N.CacheCleanupStats._fields_}

    def gc_stale_inflight(self, max_age_seconds: float) -> int:
        """Drop blocks that have waited longer than `max_age_seconds` for slots that never came (lib.rs:938-948);
        returns how many."""
        n = N.sz()
        N.check(N.lib.pf_engine_gc_stale_inflight(self._h, float(max_age_seconds), C.byref(n)))
        return int(n.value)

    def phase_times(self) -> dict:
        """{phase name: (seconds, samples)} accumulated since the engine was created; phases the
        reference traces carry its span names (``save.pinned_alloc``, ``gpu.save_task``, ...)."""
        t = N.PhaseTimes()
        N.check(N.lib.pf_engine_get_phase_times(self._h, C.byref(t)))
        return {N.lib.pf_engine_phase_name(i).decode(): (t.seconds[i], t.calls[i]) for i in range(N.PHASE_COUNT)}

    def block_slot_image(self, instance_id, raw_hash: bytes, slot: int, group: int = 0):
        """Host image of one stored slot, or None when the block is not resident."""
        (b,) = self.query_group_membership(instance_id, group, [raw_hash])
        return None if b is None else b.slot_image(slot)
