"""ctypes declarations for ``libpegaflow_b200.so`` (include/pegaflow_b200.h).

There is no Python or CPU fallback: if the shared library has not been built the import of
this module raises, and every entry point that moves bytes fails without a CUDA device.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libpegaflow_b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python pegaflow_b200/build.py` (needs nvcc; there is no CPU fallback)")

lib = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)

PF_OK = 0
STATUS_NAMES = {1: "InstanceMissing", 2: "WorkerMissing", 3: "InvalidArgument", 4: "CudaInit", 5: "Storage",
                6: "Poisoned", 7: "TopologyMismatch"}
PF_NO_BLOCK = C.c_size_t(-1).value
ROUTE_AUTO, ROUTE_STAGED, ROUTE_ZEROCOPY = 0, 1, 2
NOALLOC_MAX_PAYLOAD_BYTES = 8 << 20
NOALLOC_MAX_BLOCKS = 16384

sz = C.c_size_t
u64 = C.c_uint64
u32 = C.c_uint32
vp = C.c_void_p


class Layout(C.Structure):
    _fields_ = [("data_ptr", u64), ("size_bytes", sz), ("num_blocks", sz), ("block_stride_bytes", sz),
                ("segment_bytes", sz), ("segments", sz), ("padded_segment_bytes", sz), ("split", C.c_int),
                ("kv_stride_bytes", sz)]


class CopyDesc(C.Structure):
    _fields_ = [("device", u64), ("host", vp), ("host_device", u64), ("size", sz), ("device_allocation", sz),
                ("host_allocation", sz)]


class BackendConfig(C.Structure):
    _fields_ = [("staging_slot_bytes", sz), ("staging_slots", C.c_int), ("pack_ctas", C.c_int),
                ("link_ctas", C.c_int), ("min_dma_bytes", sz), ("route", C.c_int), ("time_kernels", C.c_int),
                ("copy_streams", C.c_int), ("gather_slots", C.c_int)]


class HostRun(C.Structure):
    _fields_ = [("first_block", sz), ("n_blocks", sz), ("host", vp), ("host_device", u64), ("stride_bytes", sz)]


class LayerXfer(C.Structure):
    _fields_ = [("data_ptr", u64), ("block_stride_bytes", sz), ("kv_stride_bytes", sz), ("range_bytes", sz),
                ("n_ranges", u32), ("n_blocks", sz), ("block_ids", C.POINTER(u32)), ("n_runs", sz * 2),
                ("runs", C.POINTER(HostRun) * 2)]


class DeviceLayout(C.Structure):
    _fields_ = [("data_ptr", u64), ("block_stride_bytes", sz), ("kv_stride_bytes", sz), ("range_bytes", sz),
                ("n_ranges", u32), ("num_blocks", sz)]


class BackendStats(C.Structure):
    _fields_ = [("kernel_launches", u64), ("dma_copies", u64), ("bytes_staged", u64), ("bytes_zero_copy", u64),
                ("bytes_peer", u64), ("device_status", u32), ("pack_kernel_ms", C.c_double),
                ("pack_kernel_launches", u64), ("pack_kernel_bytes", u64), ("link_kernel_ms", C.c_double),
                ("link_kernel_launches", u64), ("link_kernel_bytes", u64), ("pack_kernel_device_ms", C.c_double),
                ("pack_kernel_device_launches", u64)]


class PoolConfig(C.Structure):
    _fields_ = [("use_hugepages", C.c_int), ("use_mmap", C.c_int), ("numa_node", C.c_int), ("unit_hint", u64),
                ("shards", C.c_int), ("transparent_huge", C.c_int)]


class StorageConfig(C.Structure):
    _fields_ = [("enable_numa_affinity", C.c_int), ("blockwise_alloc", C.c_int), ("hint_value_size", u64),
                ("pool_shards", C.c_int), ("host_alignment", sz), ("use_mmap_pool", C.c_int),
                ("backend", BackendConfig)]


class LayerSave(C.Structure):
    _fields_ = [("layer_name", C.c_char_p), ("n_blocks", sz), ("block_ids", C.POINTER(sz)),
                ("block_hashes", C.POINTER(C.POINTER(C.c_uint8))), ("block_hash_lens", C.POINTER(sz))]


class LeaseLoad(C.Structure):
    _fields_ = [("lease", C.c_uint8 * 16), ("n_blocks", sz), ("dst_ids", C.POINTER(C.POINTER(sz)))]


class LayerGroups(C.Structure):
    _fields_ = [("n_groups", sz), ("group_sizes", C.POINTER(sz)), ("layer_names", C.POINTER(C.c_char_p))]


class EngineMetrics(C.Structure):
    _fields_ = [("save_bytes", u64), ("save_duration_seconds", C.c_double), ("save_batches", u64),
                ("load_bytes", u64), ("load_duration_seconds", C.c_double), ("load_tasks", u64),
                ("load_failures", u64), ("pool_capacity_bytes", u64), ("pool_used_bytes", u64),
                ("pool_alloc_failures", u64), ("cache_blocks", u64), ("evicted_blocks", u64),
                ("transfer", BackendStats)]


PHASE_COUNT = 17


class PhaseTimes(C.Structure):
    _fields_ = [("seconds", C.c_double * PHASE_COUNT), ("calls", u64 * PHASE_COUNT)]


def _sig(name, restype, *argtypes):
    fn = getattr(lib, name)
    fn.restype = restype
    fn.argtypes = list(argtypes)
    return fn


P = C.POINTER
_sig("pf_abi_version", C.c_int)
_sig("pf_last_error", C.c_char_p)
_sig("pf_layout_init", C.c_int, P(Layout), u64, sz, sz, sz, sz, sz, sz, sz)
_sig("pf_layout_block_copies", C.c_int, P(Layout), sz, P(u64), P(sz), P(C.c_int))
_sig("pf_build_page_layout", C.c_int, P(sz), P(sz), sz, sz, P(sz), P(sz), P(sz), P(sz), P(sz), P(sz))
_sig("pf_pool_unit_size", u64, u64, u64)
_sig("pf_backend_new", C.c_int, C.c_int, P(BackendConfig), P(vp))
_sig("pf_backend_free", None, vp)
_sig("pf_backend_name", C.c_char_p, vp)
_sig("pf_backend_h2d", C.c_int, vp, P(CopyDesc), sz, vp)
_sig("pf_backend_d2h", C.c_int, vp, P(CopyDesc), sz, vp)
_sig("pf_backend_save_layers", C.c_int, vp, P(LayerXfer), sz, vp, P(vp))
_sig("pf_backend_load_layers", C.c_int, vp, P(LayerXfer), sz, vp, P(vp))
_sig("pf_backend_gather_layers", C.c_int, vp, P(LayerXfer), sz, vp)
_sig("pf_backend_peer_copy", C.c_int, vp, P(DeviceLayout), P(u32), P(DeviceLayout), P(u32), sz, vp)
_sig("pf_backend_peer_copy_layers", C.c_int, vp, P(DeviceLayout), P(DeviceLayout), sz, P(u32), P(u32), sz, vp)
class IpcRegion(C.Structure):
    _fields_ = [("handle", C.c_uint8 * 64), ("offset", u64), ("nbytes", u64), ("device_uuid", C.c_uint8 * 16)]


_sig("pf_ipc_export", C.c_int, u64, sz, P(IpcRegion))
_sig("pf_ipc_open", C.c_int, P(IpcRegion), P(u64), P(C.c_int))
_sig("pf_ipc_close", C.c_int, P(IpcRegion))
_sig("pf_ipc_open_for", C.c_int, P(IpcRegion), C.c_int, P(u64), P(C.c_int))
_sig("pf_ipc_close_for", C.c_int, P(IpcRegion), C.c_int)
_sig("pf_enable_peer_access", C.c_int, C.c_int, C.c_int)
_sig("pf_save_blocks_noalloc", C.c_int, C.c_int, P(DeviceLayout), P(u32), sz, vp, sz, vp)
_sig("pf_backend_get_stats", C.c_int, vp, P(BackendStats))
_sig("pf_pool_new", C.c_int, sz, P(PoolConfig), P(vp))
_sig("pf_pool_free", None, vp)
_sig("pf_pool_alloc", C.c_int, vp, sz, P(vp), P(u64), P(u64))
_sig("pf_pool_release", C.c_int, vp, u64)
_sig("pf_pool_usage", C.c_int, vp, P(u64), P(u64), P(u64))
_sig("pf_numa_node_of_device", C.c_int, C.c_int)
_sig("pf_numa_num_nodes", C.c_int)
_sig("pf_numa_set_sysfs_root", C.c_int, C.c_char_p)
_sig("pf_numa_parse_cpulist", C.c_int, C.c_char_p, P(C.c_int), sz, P(sz))
_sig("pf_numa_cpus_of_node", C.c_int, C.c_int, P(C.c_int), sz, P(sz))
_sig("pf_numa_pin_thread_to_node", C.c_int, C.c_int)
_sig("pf_numa_node_of_pci_device", C.c_int, C.c_char_p)
_sig("pf_numa_parse_closest_cpu_node", C.c_int, C.c_char_p)
_sig("pf_numa_distinct_valid_nodes", C.c_int, P(C.c_int), sz, P(C.c_int), P(sz))
_sig("pf_numa_query_pages", C.c_int, P(vp), sz, P(C.c_int))
_sig("pf_pool_pre_touch_threads", sz, sz)
_sig("pf_huge_page_size", sz)
_sig("pf_engine_new", C.c_int, sz, C.c_int, P(StorageConfig), P(vp))
_sig("pf_engine_free", None, vp)
_sig("pf_engine_register_context_layer_batch_strided", C.c_int, vp, C.c_char_p, C.c_char_p, C.c_int, sz, sz, sz,
     sz, sz, P(C.c_char_p), P(u64), P(sz), P(sz), P(sz), P(sz), P(sz), P(sz), P(u32), C.c_int, C.c_int)
_sig("pf_engine_unregister_instance", C.c_int, vp, C.c_char_p)
_sig("pf_engine_batch_save", C.c_int, vp, C.c_char_p, sz, sz, C.c_int, sz, P(LayerSave))
_sig("pf_engine_flush_saves", C.c_int, vp)
_sig("pf_engine_query_prefix", C.c_int, vp, C.c_char_p, C.c_char_p, sz, P(P(C.c_uint8)), P(sz), P(vp), P(sz),
     P(sz))
_sig("pf_engine_query_group_membership", C.c_int, vp, C.c_char_p, u32, sz, P(P(C.c_uint8)), P(sz), P(vp))
_sig("pf_block_release", None, vp)
_sig("pf_blocks_release", None, P(vp), sz)
_sig("pf_block_num_slots", sz, vp)
_sig("pf_block_slot_info", C.c_int, vp, sz, P(sz), P(sz))
_sig("pf_block_slot_read", C.c_int, vp, sz, sz, vp, sz)
_sig("pf_engine_create_query_lease", C.c_int, vp, C.c_char_p, sz, P(vp), P(C.c_uint8))
_sig("pf_engine_release_query_lease", C.c_int, vp, P(C.c_uint8), P(C.c_int))
_sig("pf_engine_batch_load_shm", C.c_int, vp, C.c_char_p, sz, C.c_int, C.c_char_p, P(LayerGroups), sz,
     P(LeaseLoad))
_sig("pf_engine_batch_load_inproc", C.c_int, vp, C.c_char_p, sz, C.c_int, P(LayerGroups), sz, P(LeaseLoad), P(vp))
_sig("pf_completion_poll", C.c_int, vp, P(C.c_int))
_sig("pf_completion_wait", C.c_int, vp, C.c_double, P(C.c_int))
_sig("pf_completion_error", C.c_char_p, vp)
_sig("pf_completion_free", None, vp)
_sig("pf_engine_layer_load_event", C.c_int, vp, C.c_char_p, C.c_int, C.c_char_p, P(vp))
_sig("pf_stream_wait_event", C.c_int, vp, vp)
_sig("pf_engine_save_layers_async", C.c_int, vp, C.c_char_p, sz, sz, C.c_int, sz, P(LayerSave), vp)
_sig("pf_engine_peer_load", C.c_int, vp, C.c_char_p, C.c_int, C.c_char_p, C.c_int, sz, P(sz), P(sz))
_sig("pf_engine_list_instances", C.c_int, vp, C.c_char_p, sz, P(sz))
_sig("pf_engine_unregister_all_instances", C.c_int, vp, C.c_char_p, sz, P(sz))
_sig("pf_engine_instance_namespace", C.c_int, vp, C.c_char_p, C.c_char_p, sz, P(sz))
_sig("pf_engine_get_metrics", C.c_int, vp, P(EngineMetrics))


class CacheCleanupStats(C.Structure):
    _fields_ = [("evicted_blocks", u64), ("evicted_bytes", u64), ("reclaimed_bytes", u64), ("still_referenced_blocks", u64)]


_sig("pf_engine_cleanup_memory_cache", C.c_int, vp, P(CacheCleanupStats))
_sig("pf_engine_gc_stale_inflight", C.c_int, vp, C.c_double, P(sz))
_sig("pf_engine_get_phase_times", C.c_int, vp, P(PhaseTimes))
_sig("pf_engine_phase_name", C.c_char_p, C.c_int)
_sig("pf_load_state_new", C.c_int, P(vp))
_sig("pf_load_state_attach", C.c_int, C.c_char_p, P(vp))
_sig("pf_load_state_shm_name", C.c_char_p, vp)
_sig("pf_load_state_get", C.c_int64, vp)
_sig("pf_load_state_set_completed", None, vp)
_sig("pf_load_state_set_error", None, vp)
_sig("pf_load_state_free", None, vp)


class PegaFlowError(Exception):
    """Base error of the bindings (python/src/lib.rs:65-72 of the reference)."""

    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status
        self.kind = STATUS_NAMES.get(status, f"status {status}")


class PegaflowInternal(PegaFlowError):
    """CudaInit / Storage / Poisoned failures (gRPC INTERNAL in the reference's service)."""


class PegaflowInvalidArgument(PegaFlowError, ValueError):
    """InvalidArgument failures; the reference's bindings raise ValueError for these."""


def check(status: int):
    if status == PF_OK:
        return
    msg = lib.pf_last_error().decode(errors="replace")
    if status == 3:
        raise PegaflowInvalidArgument(status, msg)
    if status in (4, 5, 6):
        raise PegaflowInternal(status, msg)
    raise PegaFlowError(status, msg)


def release(fn_name: str, handle, _module_dict=globals()) -> None:
    """Call a `*_free` / `*_release` entry point from `close()` or `__del__`.  During interpreter
    shutdown module globals are set to None one by one while finalizers still run; the module
    dictionary is bound at definition time, and a library that is already gone means the handle is
    left to the process exit."""
    library = _module_dict.get("lib")
    if library is None:
        return
    getattr(library, fn_name)(handle)
