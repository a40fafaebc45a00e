"""Host-side mirror of the reference's worker connector surface for the save/load path.

* ``infer_kv_cache_registration`` — what ``_infer_kv_cache_registration`` derives from a vLLM KV
  tensor (python/pegaflow/connector/worker.py:65-151).
* ``InProcEngineClient`` — the method names and argument order of the reference's
  ``EngineRpcClient`` (python/src/lib.rs:205-617, stubs in python/pegaflow/pegaflow.pyi), served
  by an engine in the same process through the C ABI instead of gRPC + CUDA IPC.
* ``PegaWorkerConnector`` — the worker-side hooks of ``PegaKVConnector``
  (python/pegaflow/connector/worker.py:261-929) that touch the transfer path, including real
  bodies for vLLM's per-layer hooks, which the reference leaves empty
  (worker.py:712-713,755-765).
"""
from __future__ import annotations

import os
import threading
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

from . import _native as N
from .config import CacheGroupLayout, resolve_transfer_backend  # noqa: F401  (resolve_transfer_backend is re-exported)
from .engine import PegaEngine, PyLoadState

CROSS_LAYER_KEY = "ALL_LAYERS"  # worker.py:32


@dataclass(frozen=True)
class KVCacheRegistrationInfo:
    layout: str  # "KV-first" | "blocks-first"
    num_blocks: int
    bytes_per_block: int
    kv_stride_bytes: int
    segments: int
    physical_blocks_per_logical_block: int


def infer_kv_cache_registration(kv_cache, logical_block_size: int, *, is_mla: bool = False,
                                is_recurrent_state: bool = False) -> KVCacheRegistrationInfo:
    """Registration of one layer from its KV tensor's shape / stride / element size.

    Non-MLA tensors whose first dimension is 2 are "KV-first" (K and V regions, two segments per
    block); everything else is "blocks-first" (one segment per block).  MLA caches group the
    kernel's physical rows into scheduler-sized logical blocks.  Errors carry the reference's text.
    """
    shape = tuple(kv_cache.shape)
    stride = tuple(kv_cache.stride())
    es = kv_cache.element_size()
    if logical_block_size <= 0:
        raise ValueError(f"logical block size must be > 0, got {logical_block_size}")
    if is_recurrent_state or not is_mla:
        kv_first = (not is_recurrent_state) and len(shape) >= 2 and shape[0] == 2
        block_dim = 1 if kv_first else 0
        num_blocks = shape[block_dim]
        bytes_per_block = stride[block_dim] * es
        if num_blocks <= 0:
            raise ValueError(f"physical block count must be > 0, got {num_blocks}")
        if bytes_per_block == 0:
            raise ValueError(f"Invalid bytes_per_block: shape={shape} stride={stride}")
        return KVCacheRegistrationInfo("KV-first" if kv_first else "blocks-first", num_blocks, bytes_per_block,
                                       stride[0] * es if kv_first else 0, 2 if kv_first else 1, 1)
    rows = shape[0]
    row_tokens = shape[1] if len(shape) >= 2 else logical_block_size
    if rows <= 0:
        raise ValueError(f"physical block count must be > 0, got {rows}")
    if row_tokens <= 0:
        raise ValueError(f"physical block size must be > 0, got {row_tokens}")
    if logical_block_size % row_tokens:
        raise ValueError("logical block size must be a multiple of physical block size "
                         f"(logical={logical_block_size}, physical={row_tokens})")
    ratio = logical_block_size // row_tokens
    if rows % ratio:
        raise ValueError("physical block count must be divisible by physical/logical split ratio "
                         f"(physical_blocks={rows}, ratio={ratio})")
    bytes_per_block = stride[0] * es * ratio
    if bytes_per_block == 0:
        raise ValueError(f"Invalid bytes_per_block: shape={shape} stride={stride}")
    return KVCacheRegistrationInfo("blocks-first", rows // ratio, bytes_per_block, 0, 1, ratio)


class QueryLoading:
    """A backing-store fetch is in progress (never returned here: there is no SSD/RDMA tier)."""


@dataclass
class QueryReady:
    num_hit_blocks: int
    lease: bytes
    hit_positions: List[int] = field(default_factory=list)


def _region_of(obj) -> Tuple[int, int]:
    """(data_ptr, nbytes) of what a worker registers for one layer: a CUDA tensor (its whole
    storage, like the reference's IPC wrapper, ipc_wrapper.py:101-163) or an explicit pair."""
    if isinstance(obj, tuple):
        return int(obj[0]), int(obj[1])
    if isinstance(obj, (bytes, bytearray)):
        # the reference's `wrapper_bytes_list`: a pickled IPC wrapper from a worker in another process
        from .ipc import CudaIPCWrapper

        obj = CudaIPCWrapper.from_bytes(bytes(obj))
    if hasattr(obj, "region") and hasattr(obj, "open"):
        ptr, nbytes, _device = obj.open()
        return ptr, nbytes
    if obj.storage_offset() != 0:
        raise ValueError("KV cache tensor must have zero storage offset")
    return obj.data_ptr(), obj.untyped_storage().nbytes()


class InProcEngineClient:
    """``EngineRpcClient`` without the wire: same methods, same argument order, ``(ok, message)``
    results; invalid requests raise ``ValueError`` as the reference's bindings do."""

    def __init__(self, engine: PegaEngine):
        self._engine = engine

    def endpoint(self) -> str:
        return "inproc://pegaflow_b200"

    def health(self) -> Tuple[bool, str]:
        return True, "ok"

    @staticmethod
    def _reply(fn) -> Tuple[bool, str]:
        try:
            fn()
            return True, ""
        except N.PegaflowInvalidArgument:
            raise
        except N.PegaFlowError as e:
            return False, str(e)

    def register_context_batch(self, instance_id, namespace, tp_rank, pp_rank, tp_size, world_size, device_id,
                               layer_names, tensors, num_blocks_list, bytes_per_block_list, kv_stride_bytes_list,
                               segments_list, transfer_backend, page_first, layer_group_ids=None):
        if transfer_backend not in ("direct", "kernel"):
            raise ValueError(f"unknown transfer_backend {transfer_backend!r}")
        regions = [_region_of(t) for t in tensors]
        return self._reply(lambda: self._engine.register_context_layer_batch_strided(
            instance_id, namespace, device_id, tp_rank, pp_rank, tp_size, world_size, list(layer_names),
            [r[0] for r in regions], [r[1] for r in regions], list(num_blocks_list), list(bytes_per_block_list),
            list(kv_stride_bytes_list), list(segments_list), None,
            list(layer_group_ids) if layer_group_ids is not None else None, transfer_backend, page_first))

    def unregister_context(self, instance_id):
        return self._reply(lambda: self._engine.unregister_instance(instance_id))

    def save(self, instance_id, tp_rank, pp_rank, device_id, saves):
        return self._reply(lambda: self._engine.batch_save(instance_id, tp_rank, pp_rank, device_id, saves))

    def save_async(self, instance_id, tp_rank, pp_rank, device_id, saves, ready_event: int = 0):
        """Additive: returns once the save is queued; it starts when ``ready_event`` has fired."""
        return self._reply(lambda: self._engine.save_layers_async(instance_id, tp_rank, pp_rank, device_id, saves,
                                                                  ready_event))

    def flush_saves(self):
        return self._reply(self._engine.flush_saves)

    def load(self, instance_id, tp_rank, device_id, load_state_shm, layer_groups, loads):
        return self._reply(lambda: self._engine.batch_load_shm(instance_id, tp_rank, device_id, load_state_shm,
                                                               layer_groups, loads))

    def query_prefetch(self, instance_id, block_hashes, req_id, wait_for_full_prefix=False, group_id=0):
        if not req_id:
            raise ValueError("req_id must be non-empty")
        if group_id == 0:
            blocks, _missing = self._engine.query_prefix(instance_id, block_hashes, req_id)
            positions = list(range(len(blocks)))
        else:
            found = self._engine.query_group_membership(instance_id, group_id, block_hashes)
            positions = [i for i, b in enumerate(found) if b is not None]
            blocks = [found[i] for i in positions]
        if not blocks:
            return QueryReady(0, b"", [])
        lease = self._engine.create_query_lease(instance_id, blocks)
        return QueryReady(len(blocks), lease, positions)

    def release(self, lease: bytes) -> None:
        if lease:
            self._engine.release_query_lease(lease)

    def shutdown(self):
        return True, ""

    def start_session_watcher(self, instance_id, namespace, tp_size, world_size) -> None:
        """The reference opens a liveness stream here so that a server outliving the worker releases
        its CUDA IPC mappings (python/src/lib.rs:591-617).  The engine lives and dies with this process:
        there is nothing to watch."""
        if not instance_id:
            raise ValueError("instance_id must be non-empty")


class ServiceStateManager:
    """Whether the engine behind ``client`` is believed to be usable (state_manager.py:21-99).  The
    worker marks it unavailable when a load cannot be submitted or times out; from then on a daemon
    thread asks ``client.health()`` every ``health_check_interval`` seconds and the first healthy
    answer makes the service available again.  Load and save calls do not consult the flag — as in
    the reference it is there for whoever decides whether to look the cache up at all."""

    def __init__(self, engine_client, health_check_interval: float = 10.0):
        self._client = engine_client
        self._interval = health_check_interval
        self._lock = threading.Lock()
        self._available = True
        self._stop = threading.Event()
        self._probe: Optional[threading.Thread] = None
        self.last_reason = ""

    def is_available(self) -> bool:
        with self._lock:
            return self._available

    def mark_unavailable(self, reason: str) -> None:
        with self._lock:
            if not self._available:
                return
            self._available = False
            self.last_reason = reason
            if self._probe is None or not self._probe.is_alive():
                self._stop.clear()
                self._probe = threading.Thread(target=self._probe_until_healthy, daemon=True, name="PegaHealthCheck")
                self._probe.start()

    def _probe_until_healthy(self) -> None:
        while not self._stop.wait(self._interval):
            try:
                ok, _ = self._client.health()
            except Exception:
                continue
            if ok:
                with self._lock:
                    self._available = True
                return

    def shutdown(self) -> None:
        self._stop.set()
        probe = self._probe
        if probe is not None and probe.is_alive():
            probe.join(timeout=1.0)


def plan_group_loads(load_intents, cache_groups: CacheGroupLayout, shard_index: int = 0, shard_count: int = 1):
    """Turn the scheduler's load intents into the engine's load requests for one TP shard when the model
    has several cache groups (worker.py:571-617).  Returns (loads, destination block ids, request ids);
    a load is (lease, destination ids per cache group, `None` = skip that block).

    The prefix lease pins attention blocks only, so under it the recurrent groups get no destination.
    Each recurrent group's state travels under its own membership lease, which pins the blocks at
    `hit_positions`; only the checkpoint among them has a destination — the last block the
    scheduler allocated for that group."""
    loads, all_ids, request_ids = [], [], []
    recurrent = sorted(cache_groups.recurrent_group_indices)
    for req_id, intent in load_intents.items():
        if len(intent.leases) != shard_count:
            raise RuntimeError(f"load intent has {len(intent.leases)} TP shard leases; expected {shard_count}")
        by_group = [list(g) for g in intent.block_ids_by_group]
        hold = getattr(intent, "recurrent_hold", None)
        if hold is not None:
            for g in recurrent:
                by_group[g] = [None] * len(by_group[g])
        for ids in by_group:
            all_ids.extend(b for b in ids if b is not None)
        loads.append((intent.leases[shard_index], by_group))
        if hold is not None:
            for slot, g in enumerate(recurrent):
                positions = hold.hit_positions[slot][shard_index]
                if hold.checkpoint not in positions:
                    raise RuntimeError(f"req {req_id}: recurrent group {g} shard {shard_index} lease has no checkpoint "
                                       f"at query position {hold.checkpoint}")
                destination = next((b for b in reversed(intent.block_ids_by_group[g]) if b is not None), None)
                if destination is None:
                    raise RuntimeError(f"req {req_id}: no recurrent destination block in group {g} for checkpoint "
                                       f"{hold.checkpoint}")
                vectors = [[None] * len(positions) for _ in range(cache_groups.group_count)]
                vectors[g][list(positions).index(hold.checkpoint)] = destination
                loads.append((hold.leases[slot][shard_index], vectors))
                all_ids.append(destination)
        request_ids.append(req_id)
    return loads, all_ids, request_ids


def _load_timeout_seconds() -> int:
    """worker.py:34-43: PEGA_LOAD_TIMEOUT_SECONDS, default 120, never below 30; an unparsable value
    falls back to the default (common.py:464-485)."""
    raw = os.environ.get("PEGA_LOAD_TIMEOUT_SECONDS")
    try:
        seconds = 120 if raw is None else int(raw)
    except ValueError:
        seconds = 120
    return max(seconds, 30)


@dataclass
class _PendingLoad:
    state: PyLoadState
    request_ids: List[str]
    block_ids: List[int]
    started: float = 0.0


class TransferStats:
    """What the worker reports about its transfers between two readings, under the keys of the
    reference's ``PegaKVConnectorStats`` (connector_metrics.py:115-260): per-operation durations
    (seconds) and block counts as lists, success and failure counters, and the number of requests
    whose saves are still pending.  ``aggregate`` adds another reading to this one, ``reduce`` gives
    the summary the reference logs."""

    LISTS = ("load_duration", "load_blocks", "save_duration", "save_blocks")
    COUNTERS = ("load_success_count", "load_failure_count", "save_success_count", "save_failure_count")

    def __init__(self):
        self.reset()

    def reset(self):
        self.data = {"pending_save_requests": 0}
        self.data.update({k: [] for k in self.LISTS})
        self.data.update({k: 0 for k in self.COUNTERS})

    def _record(self, kind: str, seconds: float, blocks: int, ok: bool):
        self.data[f"{kind}_duration"].append(float(seconds))
        self.data[f"{kind}_blocks"].append(int(blocks))
        self.data[f"{kind}_{'success' if ok else 'failure'}_count"] += 1

    def record_load(self, duration_seconds: float, num_blocks: int, success: bool):
        self._record("load", duration_seconds, num_blocks, success)

    def record_save(self, duration_seconds: float, num_blocks: int, success: bool):
        self._record("save", duration_seconds, num_blocks, success)

    def is_empty(self) -> bool:
        return not self.data["pending_save_requests"] and not any(self.data[k] for k in self.LISTS + self.COUNTERS)

    def aggregate(self, other: "TransferStats") -> "TransferStats":
        self.data["pending_save_requests"] = other.data.get("pending_save_requests", 0)    # a gauge: the latest
        for k in self.COUNTERS:
            self.data[k] += other.data.get(k, 0)
        for k in self.LISTS:
            self.data[k].extend(other.data.get(k, []))
        return self

    def reduce(self) -> dict:
        out = {"pending_save_requests": self.data["pending_save_requests"]}
        for kind in ("load", "save"):
            seconds, blocks = self.data[f"{kind}_duration"], self.data[f"{kind}_blocks"]
            if seconds:
                out[f"num_{kind}s"] = len(seconds)
                out[f"avg_{kind}_duration_ms"] = round(sum(seconds) / len(seconds) * 1000, 3)
                out[f"total_{kind}_blocks"] = sum(blocks)
                out[f"avg_{kind}_blocks"] = round(sum(blocks) / len(seconds), 1)
            out[f"{kind}_success_count"] = self.data[f"{kind}_success_count"]
            out[f"{kind}_failure_count"] = self.data[f"{kind}_failure_count"]
        return out

    def clone_and_reset(self) -> "TransferStats":
        old = TransferStats()
        old.data = self.data
        self.reset()
        return old


class PegaWorkerConnector:
    """Worker-side hooks on the transfer path for one GPU of one instance."""

    LOAD_TIMEOUT_SECONDS: int = _load_timeout_seconds()   # read once at import, like worker.py:185-187

    def __init__(self, client: InProcEngineClient, engine: PegaEngine, *, instance_id: str, namespace: str,
                 device_id: int, block_size: int, tp_rank: int = 0, pp_rank: int = 0, tp_size: int = 1,
                 world_size: int = 1, is_mla: bool = False, transfer_backend: Optional[str] = None,
                 page_first: Optional[bool] = None, state_manager: Optional[ServiceStateManager] = None,
                 cache_groups: Optional[CacheGroupLayout] = None, tp_shard_count: int = 1):
        self.client, self.engine = client, engine
        # one attention (or MLA) group unless a layout says otherwise (worker.py:196-197)
        self.cache_groups = cache_groups or CacheGroupLayout(((),), 0, False, frozenset(), frozenset())
        self._layer_to_group = self.cache_groups.layer_to_group()
        self.tp_shard_count = tp_shard_count
        self.state_manager = state_manager if state_manager is not None else ServiceStateManager(client)
        self.instance_id, self.namespace, self.device_id = instance_id, namespace, device_id
        self.block_size, self.is_mla = block_size, is_mla
        self.tp_rank, self.pp_rank, self.tp_size, self.world_size = tp_rank, pp_rank, tp_size, world_size
        self.transfer_backend = resolve_transfer_backend(is_mla, transfer_backend)
        self.page_first = is_mla if page_first is None else page_first
        self.registered_layers: List[str] = []
        self.registrations: Dict[str, KVCacheRegistrationInfo] = {}
        self._pending_loads: List[_PendingLoad] = []
        self._load_errors: set = set()
        self._rejected_loads: List[str] = []      # requests whose load could not even be submitted
        self.load_history: List[Tuple[float, int, bool]] = []   # (seconds, blocks, ok) per finished load task
        self.stats = TransferStats()                             # worker.py:242
        self._saves_in_flight = 0

    # worker.py:261-412
    def register_kv_caches(self, kv_caches: Dict[str, object]):
        if not kv_caches:
            raise RuntimeError("No KV cache layers were selected for registration")
        names, tensors, nb, bpb, kvs, segs = [], [], [], [], [], []
        for name, t in kv_caches.items():
            info = infer_kv_cache_registration(t, self.block_size, is_mla=self.is_mla)
            self.registrations[name] = info
            names.append(name)
            tensors.append(t)
            nb.append(info.num_blocks)
            bpb.append(info.bytes_per_block)
            kvs.append(info.kv_stride_bytes)
            segs.append(info.segments)
        if not isinstance(self.client, InProcEngineClient):
            # an engine in another process gets the tensors as pickled CUDA IPC wrappers (worker.py:326-349)
            from .ipc import CudaIPCWrapper

            tensors = [CudaIPCWrapper(t).to_bytes() for t in tensors]
        ok, msg = self.client.register_context_batch(self.instance_id, self.namespace, self.tp_rank, self.pp_rank,
                                                     self.tp_size, self.world_size, self.device_id, names, tensors,
                                                     nb, bpb, kvs, segs, self.transfer_backend, self.page_first)
        if not ok:
            raise RuntimeError(f"Register context batch failed for layers {names}: {msg}")
        self.registered_layers = names

    # worker.py:414-420
    def register_cross_layers_kv_cache(self, kv_cache):
        key = f"{CROSS_LAYER_KEY}_pp{self.pp_rank}" if self.world_size > self.tp_size else CROSS_LAYER_KEY
        self.register_kv_caches({key: kv_cache})

    @property
    def available(self) -> bool:
        return self.state_manager.is_available()

    def unregister(self):
        self.state_manager.shutdown()
        if self.registered_layers:
            self.client.unregister_context(self.instance_id)
            self.registered_layers = []

    # worker.py:549-710
    def start_load_kv(self, loads: Sequence[Tuple[str, bytes, Sequence[Optional[int]]]]):
        """loads: (request_id, lease, destination block ids) per request; one load task for all."""
        if not loads:
            return
        state = PyLoadState()
        pending = _PendingLoad(state, [r for r, _, _ in loads], [b for _, _, ids in loads for b in ids if b is not None],
                               time.perf_counter())
        try:
            ok, msg = self.client.load(self.instance_id, self.tp_rank, self.device_id, state.shm_name(),
                                       [list(self.registered_layers)], [(lease, [list(ids)]) for _, lease, ids in loads])
        except Exception as e:      # a load that cannot be submitted never raises into the model step
            ok, msg = False, str(e)
        if not ok:
            # worker.py:650-684: the leases go back, the blocks are reported invalid so that they
            # are recomputed, and the requests are reported as received so that they are not left parked
            for _, lease, _ in loads:
                try:
                    self.client.release(lease)
                except Exception:
                    pass
            self._load_errors.update(pending.block_ids)
            self._rejected_loads.extend(pending.request_ids)
            self.stats.record_load(time.perf_counter() - pending.started, len(pending.block_ids), False)   # worker.py:741-753
            self.state_manager.mark_unavailable(f"load rpc failed: {msg}")   # worker.py:659,677
            return
        self._pending_loads.append(pending)

    # worker.py:712-713 is empty in the reference
    def wait_for_layer_load(self, layer_name: str, stream: int = 0):
        """Order `stream` after the arrival of `layer_name`'s bytes of the pending load."""
        if not self._pending_loads:
            return
        ev = self.engine.layer_load_event(self.instance_id, self.device_id, layer_name)
        self.engine.stream_wait_event(stream, ev)

    # worker.py:755-765 is a stub in the reference
    def save_kv_layer(self, layer_name: str, block_ids: Sequence[int], block_hashes: Sequence[bytes],
                      ready_event: int = 0):
        keep = [(b, h) for b, h in zip(block_ids, block_hashes) if b != 0]   # block 0 is vLLM's null block
        if not keep:
            return
        ok, msg = self.client.save_async(self.instance_id, self.tp_rank, self.pp_rank, self.device_id,
                                         [(layer_name, [b for b, _ in keep], [h for _, h in keep])], ready_event)
        if not ok:
            raise RuntimeError(f"layer save failed: {msg}")
        self._saves_in_flight += 1

    # worker.py:767-929
    def wait_for_save(self, saves: Optional[Sequence[Tuple[str, Sequence[int], Sequence[bytes]]]] = None):
        """Blocking batch save of `saves` (all layers, one GPU batch), then a flush that also
        covers layer saves queued by save_kv_layer."""
        if saves:
            cleaned, memo = [], {}
            for name, ids, hashes in saves:
                if self.page_first and self.tp_size > 1:
                    # worker.py:982-1005: a page needs every layer, so page-first spreads the save work
                    # by block, not by layer: rank r writes the pages of blocks with id % tp_size == r
                    key = ("stripe", id(ids), id(hashes))
                    if key not in memo:
                        keep = [(b, h) for b, h in zip(ids, hashes) if b % self.tp_size == self.tp_rank]
                        memo[key] = ([b for b, _ in keep], [h for _, h in keep])
                    ids, hashes = memo[key]
                # layers usually share one (ids, hashes) pair: filter it once and hand the engine the
                # same list objects for every layer, so that it marshals them once as well
                key = (id(ids), id(hashes))
                if key not in memo:
                    if 0 in ids:
                        keep = [(b, h) for b, h in zip(ids, hashes) if b != 0]
                        memo[key] = ([b for b, _ in keep], [h for _, h in keep])
                    else:
                        memo[key] = (ids, hashes)
                cleaned.append((name,) + memo[key])
            started = time.perf_counter()
            try:
                ok, msg = self.client.save(self.instance_id, self.tp_rank, self.pp_rank, self.device_id, cleaned)
            except Exception:
                self.stats.record_save(time.perf_counter() - started, sum(len(ids) for _, ids, _ in cleaned), False)
                raise
            self.stats.record_save(time.perf_counter() - started, sum(len(ids) for _, ids, _ in cleaned), ok)   # worker.py:925-926
            if not ok:
                raise RuntimeError(f"save failed: {msg}")
        ok, msg = self.client.flush_saves()
        self._saves_in_flight = 0
        if not ok:
            raise RuntimeError(f"save failed: {msg}")

    # worker.py:549-560 / :767-800: the scheduler's per-step metadata drives both directions
    def start_load_kv_from_metadata(self, metadata, shard_index: int = 0):
        """Start every load the scheduler planned for this step (one lease per TP shard: this
        worker's shard consumes `leases[shard_index]`)."""
        if self.cache_groups.group_count > 1:
            return self._start_group_loads(metadata.load_intents, shard_index)
        self.start_load_kv([(req_id, intent.leases[shard_index], list(intent.block_ids_by_group[0]))
                            for req_id, intent in metadata.load_intents.items()])

    def layer_groups(self) -> List[List[str]]:
        """Registered layers by cache group, in registration order (worker.py:624-633)."""
        groups: List[List[str]] = [[] for _ in range(self.cache_groups.group_count)]
        for name in self.registered_layers:
            groups[self._layer_to_group.get(name, 0)].append(name)
        return groups

    def _start_group_loads(self, load_intents, shard_index: int):
        """Loads of a model with several cache groups (worker.py:571-684).  vLLM cannot recompute a
        failed load for several groups, so a load that cannot be submitted raises after its leases went back."""
        if not load_intents:
            return
        loads, all_ids, request_ids = plan_group_loads(load_intents, self.cache_groups, shard_index, self.tp_shard_count)
        layer_groups = self.layer_groups()
        if not all_ids or not any(layer_groups):
            return
        state = PyLoadState()
        try:
            ok, msg = self.client.load(self.instance_id, self.tp_rank, self.device_id, state.shm_name(), layer_groups, loads)
        except Exception as e:
            ok, msg = False, str(e)
        if not ok:
            for lease, _ in loads:
                try:
                    self.client.release(lease)
                except Exception:
                    pass
            self.state_manager.mark_unavailable(f"load rpc failed: {msg}")
            raise RuntimeError("PegaFlow HMA load failed; vLLM cannot recover failed loads for multiple cache groups: "
                               f"{msg}")
        self._pending_loads.append(_PendingLoad(state, request_ids, all_ids, time.perf_counter()))

    def wait_for_save_from_metadata(self, metadata):
        """Save what the scheduler marked as newly full this step: every registered layer stores the
        same block ids under the same hashes.  Returns the request ids whose saves are now in the pool
        (what the worker reports back as `finished_sending`)."""
        intents = list(metadata.ready_save_intents.items()) + list(metadata.save_intents.items())
        saves = []
        for _req_id, intent in intents:
            hashes = list(intent.block_hashes)
            per_group: Dict[int, List[int]] = {}
            for name in self.registered_layers:
                # worker.py:850-866: a layer saves the block ids of its own cache group
                g = self._layer_to_group.get(name, 0)
                if g not in per_group:
                    if g >= len(intent.block_ids_by_group):
                        raise RuntimeError(f"save intent is missing cache group {g} for {name}")
                    per_group[g] = list(intent.block_ids_by_group[g])
                    if len(per_group[g]) != len(hashes):
                        raise RuntimeError(f"save block/hash count mismatch for {name}: blocks={len(per_group[g])} "
                                           f"hashes={len(hashes)}")
                saves.append((name, per_group[g], hashes))
        self.wait_for_save(saves)
        return {req_id for req_id, _ in intents}

    # worker.py:1007-1037
    def handle_preemptions(self, preempted_req_ids) -> None:
        """Called before the blocks of preempted requests are handed to someone else: any layer save
        still queued (save_kv_layer is asynchronous) must have read them by then."""
        if preempted_req_ids and self._saves_in_flight:
            ok, msg = self.client.flush_saves()
            self._saves_in_flight = 0
            if not ok:
                raise RuntimeError(f"save failed: {msg}")

    # worker.py:422-547
    def get_finished(self) -> Tuple[List[str], List[str]]:
        """(request ids whose load finished, request ids whose load failed)."""
        done, still = [], []
        failed, self._rejected_loads = self._rejected_loads, []
        now = time.perf_counter()
        multi_group = self.cache_groups.group_count > 1
        hma_failure = None
        timed_out = False
        for p in self._pending_loads:
            st = p.state.get_state()
            if st == 0 and now - p.started <= self.LOAD_TIMEOUT_SECONDS:
                still.append(p)
                continue
            if st == 1:
                done.extend(p.request_ids)
            elif multi_group:
                # worker.py:467-470, 499-503: vLLM cannot recompute a partial load of several cache groups,
                # so such a failure is not reported as invalid blocks; it ends the step (below)
                if st == 0:
                    hma_failure = f"load timed out for requests {sorted(p.request_ids)} after {now - p.started:.1f}s"
                else:
                    hma_failure = f"async load failed for requests {sorted(p.request_ids)}: state={st}"
                done.extend(p.request_ids)
            else:
                # failed, or (worker.py:454-507) pending for longer than the timeout: the requests are
                # handed back as received and their blocks are reported invalid, so that vLLM recomputes
                # them instead of waiting for ever
                failed.extend(p.request_ids)
                self._load_errors.update(p.block_ids)
            timed_out = timed_out or st == 0
            self.load_history.append((now - p.started, len(p.block_ids), st == 1))
            self.stats.record_load(now - p.started, len(p.block_ids), st == 1)            # worker.py:525-528
        self._pending_loads = still
        del self.load_history[:-1024]
        if timed_out:
            self.state_manager.mark_unavailable("load timeout")   # worker.py:522-523
        if hma_failure is not None:
            # worker.py:534-539
            self.state_manager.mark_unavailable(hma_failure)
            raise RuntimeError("PegaFlow HMA load failed; vLLM cannot recover failed loads for multiple cache groups: "
                               f"{hma_failure}")
        return done, failed

    def get_stats(self) -> Optional[TransferStats]:
        """worker.py:1039-1047: what happened since the last reading, or None when nothing did."""
        self.stats.data["pending_save_requests"] = self._saves_in_flight
        if self.stats.is_empty():
            return None
        return self.stats.clone_and_reset()

    def get_block_ids_with_load_errors(self) -> set:
        out, self._load_errors = self._load_errors, set()
        return out
