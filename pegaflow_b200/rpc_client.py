"""``EngineRpcClient``: the worker/scheduler side of the sidecar, with the surface of the reference's
client (python/src/lib.rs:287-617, stubs in python/pegaflow/pegaflow.pyi): same method names,
argument order and results — ``(ok, message)`` tuples, ``QueryReady`` / ``QueryLoading`` — and the
same error mapping: INVALID_ARGUMENT raises ``ValueError``, INTERNAL ``PegaflowInternal``, everything
else ``PegaFlowError``; a query that cannot reach the server (UNAVAILABLE, DEADLINE_EXCEEDED) is a
zero-hit ``QueryReady`` (lib.rs:505-519).  It talks to :mod:`pegaflow_b200.server` or to a reference
server alike (same wire contract).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import grpc

from . import rpc_proto as R
from ._native import PegaFlowError, PegaflowInternal
from .connector import QueryLoading, QueryReady

pb = R.pb
_MAX = 64 << 20   # lib.rs:224-228


class _RpcInvalidArgument(PegaFlowError, ValueError):
    pass


def _raise(method: str, err: grpc.RpcError):
    msg = f"{method} RPC failed: status: {err.code().name}, message: {err.details()!r}"
    if err.code() == grpc.StatusCode.INVALID_ARGUMENT:
        raise _RpcInvalidArgument(3, msg) from None
    if err.code() == grpc.StatusCode.INTERNAL:
        raise PegaflowInternal(5, msg) from None
    raise PegaFlowError(0, msg) from None


class EngineRpcClient:
    def __init__(self, endpoint: str = "http://127.0.0.1:50055", *, timeout: Optional[float] = None,
                 client_version: str = R.PROTOCOL_VERSION):
        self._endpoint = endpoint
        target = endpoint.split("://", 1)[-1]
        self._channel = grpc.insecure_channel(target, options=[("grpc.max_receive_message_length", _MAX),
                                                               ("grpc.max_send_message_length", _MAX)])
        self._timeout = timeout
        self._version = client_version
        self._session = None
        self._calls = {}
        for name, (req, resp, streaming) in R.METHODS.items():
            make = self._channel.unary_stream if streaming else self._channel.unary_unary
            self._calls[name] = make(R.method_path(name), request_serializer=R.message_class(req).SerializeToString,
                                     response_deserializer=R.message_class(resp).FromString)

    def endpoint(self) -> str:
        return self._endpoint

    def close(self):
        if self._session is not None:
            self._session.cancel()
            self._session = None
        self._channel.close()

    def _call(self, method: str, request):
        try:
            return self._calls[method](request, timeout=self._timeout)
        except grpc.RpcError as e:
            _raise(method, e)

    @staticmethod
    def _status(resp) -> Tuple[bool, str]:
        return bool(resp.status.ok), resp.status.message

    # ---- python/src/lib.rs:287-360
    def health(self) -> Tuple[bool, str]:
        return self._status(self._call("Health", pb.HealthRequest()))

    def register_context_batch(self, instance_id, namespace, tp_rank, pp_rank, tp_size, world_size, device_id,
                               layer_names, wrapper_bytes_list, num_blocks_list, bytes_per_block_list,
                               kv_stride_bytes_list, segments_list, transfer_backend, page_first, layer_group_ids=None):
        if transfer_backend not in R.TRANSFER_MODE:
            raise ValueError(f"unknown transfer_backend {transfer_backend!r}")
        req = pb.RegisterContextRequest(
            instance_id=instance_id, namespace=namespace, tp_rank=tp_rank, tp_size=tp_size, world_size=world_size,
            device_id=device_id, layer_names=list(layer_names), wrapper_bytes=[bytes(b) for b in wrapper_bytes_list],
            num_blocks=list(num_blocks_list), bytes_per_block=list(bytes_per_block_list),
            kv_stride_bytes=list(kv_stride_bytes_list), segments=list(segments_list), pp_rank=pp_rank,
            client_version=self._version, transfer_mode=R.TRANSFER_MODE[transfer_backend], page_first=bool(page_first),
            layer_group_ids=list(layer_group_ids) if layer_group_ids is not None else [])
        return self._status(self._call("RegisterContextBatch", req))

    def unregister_context(self, instance_id):
        return self._status(self._call("UnregisterContext", pb.UnregisterRequest(instance_id=instance_id)))

    def save(self, instance_id, tp_rank, pp_rank, device_id, saves):
        req = pb.SaveRequest(instance_id=instance_id, tp_rank=tp_rank, pp_rank=pp_rank, device_id=device_id,
                             saves=[pb.SaveLayer(layer_name=n, block_ids=[int(i) for i in ids],
                                                 block_hashes=[bytes(h) for h in hashes]) for n, ids, hashes in saves])
        return self._status(self._call("Save", req))

    def flush_saves(self) -> Tuple[bool, str]:
        """Saves are complete when `save` returns (the server's save is blocking): nothing to flush."""
        return True, ""

    def load(self, instance_id, tp_rank, device_id, load_state_shm, layer_groups, loads):
        def target(v):
            return pb.LoadBlockTarget() if v is None else pb.LoadBlockTarget(block_id=int(v))

        req = pb.LoadRequest(
            instance_id=instance_id, tp_rank=tp_rank, device_id=device_id, load_state_shm=load_state_shm,
            groups=[pb.LoadGroup(layer_names=list(g)) for g in layer_groups],
            loads=[pb.LeaseLoad(lease=bytes(lease), block_ids_by_group=[pb.LoadBlockIds(targets=[target(v) for v in ids])
                                                                       for ids in by_group]) for lease, by_group in loads])
        return self._status(self._call("Load", req))

    def query_prefetch(self, instance_id, block_hashes: Sequence[bytes], req_id, wait_for_full_prefix=False, group_id=0):
        req = pb.QueryRequest(instance_id=instance_id, block_hashes=[bytes(h) for h in block_hashes], req_id=req_id,
                              wait_for_full_prefix=bool(wait_for_full_prefix), group_id=group_id)
        try:
            resp = self._calls["QueryPrefetch"](req, timeout=self._timeout)
        except grpc.RpcError as e:
            if e.code() in (grpc.StatusCode.UNAVAILABLE, grpc.StatusCode.DEADLINE_EXCEEDED):
                return QueryReady(0, b"", [])      # lib.rs:505-519: an unreachable server is a miss, not an error
            _raise("query_prefetch", e)
        if resp.WhichOneof("outcome") == "loading":
            return QueryLoading()
        return QueryReady(int(resp.ready.num_hit_blocks), bytes(resp.ready.lease), list(resp.ready.hit_positions))

    def release(self, lease: bytes) -> None:
        self._call("Release", pb.ReleaseRequest(lease=bytes(lease)))

    def shutdown(self):
        return self._status(self._call("Shutdown", pb.ShutdownRequest()))

    def start_session_watcher(self, instance_id, namespace, tp_size, world_size) -> None:
        """lib.rs:591-617: open the liveness stream and hold it; when this process goes away the server
        drops the instance's CUDA IPC mappings.  Calling again replaces the previous stream."""
        if not instance_id:
            raise ValueError("instance_id must be non-empty")
        stream = self._calls["Session"](pb.SessionRequest(instance_id=instance_id, namespace=namespace, tp_size=tp_size,
                                                          world_size=world_size))
        old, self._session = self._session, stream
        if old is not None:
            old.cancel()
