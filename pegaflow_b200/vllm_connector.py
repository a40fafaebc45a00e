"""vLLM v1 KV-connector plug-in on top of this library: ``PegaKVConnector``.

Takes the place of the reference's ``pegaflow.connector.PegaKVConnector``
(python/pegaflow/connector/__init__.py) for the case this library covers: one node, attention-only
models with one KV-cache group; the engine in the vLLM process, or behind the sidecar
(``python -m pegaflow_b200.server``) like the reference's.  Configure it as

    KVTransferConfig(kv_connector="PegaKVConnector",
                     kv_connector_module_path="pegaflow_b200.vllm_connector",
                     kv_role="kv_both",
                     kv_connector_extra_config={"pegaflow.pool_bytes": 8 << 30})

Extra-config keys: ``pegaflow.pool_bytes`` (pinned pool size), ``pegaflow.mode`` ("read_write" or
"save_only", as in the reference), ``pegaflow.transfer_backend`` ("direct" or "kernel": accepted and
validated as in the reference, both served by the one transfer path here), ``pegaflow.layerwise`` (default true: loads are synchronous
from the scheduler's point of view and every attention layer waits on the stream for its own
layer's bytes, saves are queued per layer behind the layer's compute; false: the reference's
behaviour — asynchronous request-level loads, one batch save after the forward pass).

Without a server address the scheduler role and the worker role of one vLLM process share one
engine (looked up by instance id), so that form works with the in-process engine core and the
uniprocess executor (``VLLM_ENABLE_V1_MULTIPROCESSING=0``, tensor_parallel_size 1).

With ``pegaflow.host`` / ``pegaflow.port`` (or ``PEGAFLOW_HOST`` / ``PEGAFLOW_PORT``, which win, as in
connector/__init__.py:96-103) both roles talk to the sidecar over gRPC instead: the worker sends its
KV-cache tensors as CUDA IPC wrappers with its own tensor-parallel and pipeline rank, the scheduler
role queries and holds the session's liveness stream (connector/__init__.py:200-211).  That is the
reference's deployment, workers in other processes included; loads are asynchronous request-level
loads and saves one batch after the forward pass, as there (the per-layer hooks need the engine's
CUDA events in the worker's process, so ``pegaflow.layerwise`` cannot be combined with a server).
"""
from __future__ import annotations

import os
import sys
import threading
from typing import Any, Dict, Optional

import torch
from vllm.distributed.kv_transfer.kv_connector.v1.base import KVConnectorBase_V1, KVConnectorMetadata, KVConnectorRole

from . import connector as _connector
from .config import PegaConnectorMode, derive_namespace, resolve_instance_id
from .engine import PegaEngine
from .scheduler import PegaConnectorMetadata, SchedulerConnector, require_single_attention_group

_DEBUG = os.environ.get("PEGAFLOW_B200_TRACE", "0") == "1"
_ENGINES: Dict[str, PegaEngine] = {}
_ENGINES_LOCK = threading.Lock()


def shared_engine(instance_id: str, pool_bytes: int) -> PegaEngine:
    """The engine both roles of one process use."""
    with _ENGINES_LOCK:
        eng = _ENGINES.get(instance_id)
        if eng is None:
            eng = _ENGINES[instance_id] = PegaEngine(pool_bytes)
        return eng


def close_shared_engines() -> None:
    with _ENGINES_LOCK:
        for eng in _ENGINES.values():
            eng.close()
        _ENGINES.clear()


def global_device_id(local_index: int) -> int:
    """The device's index as a process without CUDA_VISIBLE_DEVICES sees it (the server), from this
    process's index among its visible devices (connector/__init__.py:475-497)."""
    visible = [v.strip() for v in os.environ.get("CUDA_VISIBLE_DEVICES", "").split(",") if v.strip()]
    if local_index < len(visible) and visible[local_index].isdigit():
        return int(visible[local_index])
    return local_index


class _Metadata(PegaConnectorMetadata, KVConnectorMetadata):
    """The scheduler connector's metadata, typed for vLLM."""


class _LocalPrefixView:
    """`KVCacheBlocks` as the scheduler connector reads it, with the locally computed prefix given
    explicitly instead of inferred from block hashes."""

    def __init__(self, blocks, local_blocks: int):
        self._blocks = blocks
        ids = blocks.get_block_ids()[0]
        self.blocks = [[_Hashed(i < local_blocks) for i in range(len(ids))]]

    def get_block_ids(self):
        return self._blocks.get_block_ids()


class _Hashed:
    __slots__ = ("block_hash",)

    def __init__(self, hashed: bool):
        self.block_hash = b"local" if hashed else None


class PegaKVConnector(KVConnectorBase_V1):
    def __init__(self, vllm_config, role: KVConnectorRole, kv_cache_config=None):
        super().__init__(vllm_config, role, kv_cache_config)
        require_single_attention_group(kv_cache_config)
        cfg = vllm_config.kv_transfer_config
        extra = cfg.get_from_extra_config
        # the reference's rule (common.py:488-516); without any configured id both roles of this process
        # must still agree, so the generated-uuid fallback is replaced by a fixed name
        configured = cfg.engine_id or getattr(vllm_config, "instance_id", "") or os.environ.get("PEGAFLOW_INSTANCE_ID")
        self._instance_id = resolve_instance_id(vllm_config) if configured else "vllm"
        self._block_size = vllm_config.cache_config.block_size
        host = os.environ.get("PEGAFLOW_HOST") or extra("pegaflow.host", None)
        port = os.environ.get("PEGAFLOW_PORT") or extra("pegaflow.port", None)
        self._remote = host is not None or port is not None
        self._layerwise = bool(extra("pegaflow.layerwise", not self._remote))
        if self._remote and self._layerwise:
            raise ValueError("pegaflow.layerwise needs the engine in the vLLM process: it cannot be combined with "
                             "pegaflow.host / pegaflow.port")
        self._read_enabled = PegaConnectorMode.from_config(extra("pegaflow.mode", "read_write")) is PegaConnectorMode.READ_WRITE
        model = vllm_config.model_config
        # every factor that changes a stored block's layout, hashed as the reference does (common.py:519-565)
        self._namespace = derive_namespace(vllm_config, vllm_config.parallel_config.tensor_parallel_size)
        self._is_mla = bool(getattr(model, "use_mla", False))
        # Scheduler and worker share one in-process engine and the worker registers as rank 0 of 1: with
        # several workers every one of them would save into a private pool as rank 0 and every lookup
        # would miss.  Refused like the group layouts this plug-in cannot serve.
        parallel = vllm_config.parallel_config
        tp_size = int(getattr(parallel, "tensor_parallel_size", 1) or 1)
        world_size = int(getattr(parallel, "world_size", 1) or 1)
        n_workers = world_size * int(getattr(parallel, "data_parallel_size", 1) or 1)
        if self._remote:
            from .rpc_client import EngineRpcClient

            self._engine = None
            self._client = EngineRpcClient(f"{host or 'http://127.0.0.1'}:{port or 50055}")
        else:
            if n_workers > 1:
                raise ValueError(
                    "pegaflow_b200's vLLM plug-in with the engine in the vLLM process runs scheduler and worker in one "
                    f"process with one worker (tensor/pipeline/data parallel world of 1); this configuration has {n_workers} "
                    "workers: start the sidecar and set pegaflow.host / pegaflow.port")
            self._engine = shared_engine(self._instance_id, int(extra("pegaflow.pool_bytes", 4 << 30)))
            self._client = _connector.InProcEngineClient(self._engine)
        self._scheduler: Optional[SchedulerConnector] = None
        self._worker: Optional[_connector.PegaWorkerConnector] = None
        if role == KVConnectorRole.SCHEDULER:
            self._scheduler = SchedulerConnector([self._client], instance_id=self._instance_id, block_size=self._block_size,
                                                 read_enabled=self._read_enabled)
            if self._remote:
                # one liveness stream per vLLM replica, from the scheduler's process: when it goes away the
                # server drops the instance and its CUDA IPC mappings (connector/__init__.py:200-211)
                self._client.start_session_watcher(self._instance_id, self._namespace, tp_size, world_size)
        else:
            device = torch.cuda.current_device()
            ranks = {}
            if self._remote:
                from vllm.distributed.parallel_state import get_pp_group, get_tensor_model_parallel_rank

                device = global_device_id(device)
                ranks = dict(tp_rank=get_tensor_model_parallel_rank(), pp_rank=get_pp_group().rank_in_group,
                             tp_size=tp_size, world_size=world_size)
            self._worker = _connector.PegaWorkerConnector(
                self._client, self._engine, instance_id=self._instance_id, namespace=self._namespace, device_id=device,
                block_size=self._block_size, is_mla=self._is_mla, **ranks,
                # "direct" / "kernel", validated like the reference (common.py:577-594); both name this library's
                # one transfer path
                transfer_backend=extra("pegaflow.transfer_backend", None))
            self._saved_requests: set = set()      # requests with saves in the pool, not yet reported sent
            self._events = []                      # per-layer "KV written" events of the current step
            self._layers_queued: set = set()       # layers whose save_kv_layer hook ran in the current step
            self._loading_this_step = False

    @classmethod
    def requires_piecewise_for_cudagraph(cls, extra_config) -> bool:
        # the per-layer hooks are Python between attention layers: a full CUDA graph would skip them
        return bool((extra_config or {}).get("pegaflow.layerwise", True))

    # ================================================================== scheduler role
    def get_num_new_matched_tokens(self, request, num_computed_tokens):
        tokens, load_async = self._scheduler.get_num_new_matched_tokens(request, num_computed_tokens)
        if _DEBUG:
            print(f"[pegaflow_b200] lookup {request.request_id}: local={num_computed_tokens} "
                  f"hashes={len(request.block_hashes)} tokens={request.num_tokens} -> {tokens}", file=sys.stderr)
        if tokens and self._layerwise:
            # The request is scheduled in this very step; its attention layers wait for their own
            # layer's bytes (wait_for_layer_load), so nothing has to be parked in the scheduler.
            load_async = False
        return tokens, load_async

    def update_state_after_alloc(self, request, blocks, num_external_tokens):
        if self._layerwise and num_external_tokens > 0:
            # With a synchronous load vLLM has already given every full block its hash, the ones
            # about to be loaded included, so "blocks that carry a hash" no longer means "computed
            # locally": the local prefix is where the lookup started.
            local = self._scheduler.pending_lookup_position(request.request_id)
            if local is not None:
                blocks = _LocalPrefixView(blocks, local)
        self._scheduler.update_state_after_alloc(request, blocks, num_external_tokens)

    def build_connector_meta(self, scheduler_output) -> KVConnectorMetadata:
        meta = self._scheduler.build_connector_meta(scheduler_output)
        return _Metadata(meta.load_intents, meta.save_intents, meta.ready_save_intents, meta.preempted_req_ids)

    def update_connector_output(self, connector_output):
        self._scheduler.update_connector_output(connector_output)

    def request_finished(self, request, block_ids):
        return self._scheduler.request_finished(request, (block_ids,))

    # ================================================================== worker role
    def register_kv_caches(self, kv_caches: Dict[str, torch.Tensor]):
        self._worker.register_kv_caches(kv_caches)

    def handle_preemptions(self, kv_connector_metadata) -> None:
        if self._worker is not None:
            self._worker.handle_preemptions(getattr(kv_connector_metadata, "preempted_req_ids", None))

    def start_load_kv(self, forward_context, **kwargs: Any) -> None:
        meta = self._get_connector_metadata()
        self._loading_this_step = bool(meta.load_intents)
        if meta.load_intents:
            # layer-wise: this step's forward pass consumes the blocks, layer by layer, on the compute
            # stream (wait_for_layer_load); otherwise the scheduler parks the requests until
            # get_finished reports them received
            self._worker.start_load_kv_from_metadata(meta)

    def wait_for_layer_load(self, layer_name: str) -> None:
        if self._layerwise and self._loading_this_step:
            self._worker.wait_for_layer_load(layer_name, torch.cuda.current_stream().cuda_stream)

    def save_kv_layer(self, layer_name: str, kv_layer, attn_metadata, **kwargs: Any) -> None:
        if not self._layerwise:
            return
        meta = self._get_connector_metadata()
        if not meta.save_intents and not meta.ready_save_intents:
            return
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream())
        self._events.append(ready)      # kept until wait_for_save: the engine waits on it from another thread
        self._layers_queued.add(layer_name)
        for intent in list(meta.ready_save_intents.values()) + list(meta.save_intents.values()):
            self._worker.save_kv_layer(layer_name, list(intent.block_ids_by_group[0]), list(intent.block_hashes),
                                       ready.cuda_event)

    def wait_for_save(self):
        meta = self._get_connector_metadata()
        wanted = bool(meta.save_intents or meta.ready_save_intents)
        if self._layerwise and not (wanted and len(self._layers_queued) < len(self._worker.registered_layers)):
            self._worker.wait_for_save()        # the layers were queued one by one: this only flushes
            self._saved_requests.update(meta.save_intents)
            self._saved_requests.update(meta.ready_save_intents)
            self._events.clear()
            self._layers_queued.clear()
        else:
            # Request-level mode - or a step whose per-layer hooks did not run for every layer (a
            # forward pass replayed from a full CUDA graph skips the Python between layers): save
            # everything after the forward pass (a layer that was queued already is copied again; the
            # first copy of a slot wins in the engine).
            self._worker.wait_for_save()
            self._events.clear()
            self._layers_queued.clear()
            torch.cuda.current_stream().synchronize()
            self._saved_requests.update(self._worker.wait_for_save_from_metadata(meta))
        self._loading_this_step = False

    def get_finished(self, finished_req_ids):
        sending = {r for r in finished_req_ids if r in self._saved_requests}
        self._saved_requests -= sending
        done, failed = self._worker.get_finished()
        # Only request-level (asynchronous) loads are parked in the scheduler and need reporting.
        receiving = None if self._layerwise else (set(done) | set(failed))
        return (sending or None), (receiving or None)

    def get_block_ids_with_load_errors(self):
        return self._worker.get_block_ids_with_load_errors()

    def shutdown(self):
        if self._scheduler is not None:
            self._scheduler.shutdown()
        if self._worker is not None:
            self._worker.unregister()
