"""The engine behind a process boundary: a gRPC sidecar with the reference's wire contract.

``serve(engine, address)`` puts a ``PegaEngine`` behind the ``pegaflow.Engine`` service
(pegaflow-server/src/service.rs:362-1072): RegisterContextBatch, Save, Load, QueryPrefetch,
Release, UnregisterContext, Health, Shutdown and the Session liveness stream.  A worker process
sends its KV-cache tensors as pickled IPC wrappers (this library's, or the reference's
``pegaflow.ipc_wrapper.CudaIPCWrapper``), the server maps them and registers the pointers, and all
bytes move on the server's GPU workers exactly as for an in-process caller.

What it keeps of the reference's behaviour:
  * status codes: InvalidArgument -> INVALID_ARGUMENT, InstanceMissing / WorkerMissing /
    TopologyMismatch -> FAILED_PRECONDITION, CudaInit / Storage / Poisoned -> INTERNAL
    (service.rs:85-96);
  * request validation and its texts (service.rs:98-165): version handshake, device id, tp sizes,
    array lengths, req_id;
  * a failed registration unmaps what it had mapped (service.rs:318-330);
  * the Session stream: when it closes, the instance's mappings are dropped and the instance is
    unregistered, unless a newer session has replaced it (session.rs, service.rs:1017-1072).
The cross-node calls (QueryBlocksForTransfer, ReleaseTransferLock, RdmaHandshake) answer
UNIMPLEMENTED: there is no RDMA tier here.
"""
from __future__ import annotations

import io
import pickle
import threading
from concurrent import futures
from typing import Dict, List, Optional, Tuple

import grpc

from . import rpc_proto as R

pb = R.pb
MAX_MESSAGE_BYTES = 64 << 20      # python/src/lib.rs:224-228, pegaflow-server/src/lib.rs:678-682


class SessionRegistry:
    """session.rs:25-80: one live session token per instance; a newer session supersedes the older,
    whose cleanup then does nothing."""

    def __init__(self):
        self._lock = threading.Lock()
        self._sessions: Dict[str, Tuple[int, Tuple[str, int, int]]] = {}
        self._next = 0

    def install(self, instance_id: str, namespace: str, tp_size: int, world_size: int) -> int:
        with self._lock:
            self._next += 1
            self._sessions[instance_id] = (self._next, (namespace, tp_size, world_size))
            return self._next

    def topology(self, instance_id: str) -> Optional[Tuple[str, int, int]]:
        with self._lock:
            entry = self._sessions.get(instance_id)
            return entry[1] if entry else None

    def take(self, instance_id: str, token: int) -> bool:
        with self._lock:
            entry = self._sessions.get(instance_id)
            if entry and entry[0] == token:
                del self._sessions[instance_id]
                return True
            return False


class _ReferenceWrapper:
    """Stand-in for the reference's ``pegaflow.ipc_wrapper.CudaIPCWrapper`` when its pickle is read
    here: the attributes are restored as they were written (ipc_wrapper.py:119-133)."""


class _WrapperUnpickler(pickle.Unpickler):
    """Wrapper bytes come from another process: only the two wrapper classes and the torch types
    they carry may be instantiated."""

    def find_class(self, module, name):
        if (module, name) == ("pegaflow_b200.ipc", "CudaIPCWrapper"):
            from .ipc import CudaIPCWrapper

            return CudaIPCWrapper
        if name == "CudaIPCWrapper" and module.startswith("pegaflow"):
            return _ReferenceWrapper
        if module in ("torch", "torch._utils", "torch.storage", "collections", "builtins", "torch.serialization"):
            return super().find_class(module, name)
        raise pickle.UnpicklingError(f"wrapper bytes may not reference {module}.{name}")


class TensorRegistry:
    """registry.rs:172-203: wrapper bytes -> (data_ptr, size_bytes), kept per registration context
    and per instance so that they can be dropped together."""

    def __init__(self):
        self._lock = threading.Lock()
        self._by_context: Dict[str, List[object]] = {}

    def register_layers(self, context_key: str, device_id: int, wrapper_bytes: List[bytes]):
        opened, out = [], []
        try:
            for raw in wrapper_bytes:
                obj = _WrapperUnpickler(io.BytesIO(raw)).load()
                if isinstance(obj, _ReferenceWrapper):
                    import torch

                    # ipc_wrapper.py:135-163: the device is found by UUID, the storage rebuilt from the handle
                    uuid = getattr(obj, "device_uuid")
                    index = next((i for i in range(torch.cuda.device_count())
                                  if str(torch.cuda.get_device_properties(i).uuid) == uuid), None)
                    if index is None:
                        raise RuntimeError(f"Device UUID {uuid} not found in the discovered devices")
                    storage = torch.UntypedStorage._new_shared_cuda(index, *obj.handle[1:])
                    opened.append(storage)
                    out.append((storage.data_ptr(), storage.nbytes()))
                else:
                    ptr, nbytes, _dev = obj.open()
                    opened.append(obj)
                    out.append((ptr, nbytes))
        except Exception:
            self._close(opened)
            raise
        with self._lock:
            self._by_context.setdefault(context_key, []).extend(opened)
        return out

    @staticmethod
    def _close(objs):
        for o in objs:
            close = getattr(o, "close", None)
            if close:
                try:
                    close()
                except Exception:
                    pass

    def drop_context(self, context_key: str) -> int:
        with self._lock:
            objs = self._by_context.pop(context_key, [])
        self._close(objs)
        return len(objs)

    def drop_instance(self, instance_id: str) -> int:
        with self._lock:
            keys = [k for k in self._by_context if k.startswith(instance_id + ":")]
            objs = [o for k in keys for o in self._by_context.pop(k)]
        self._close(objs)
        return len(objs)


def _status_of(exc) -> grpc.StatusCode:
    """service.rs:85-96 `map_engine_error`, for this library's and the oracle model's errors alike."""
    kind = getattr(exc, "kind", "")
    if kind == "InvalidArgument" or isinstance(exc, ValueError):
        return grpc.StatusCode.INVALID_ARGUMENT
    if kind in ("InstanceMissing", "WorkerMissing", "TopologyMismatch"):
        return grpc.StatusCode.FAILED_PRECONDITION
    return grpc.StatusCode.INTERNAL


class EngineService:
    """The handlers.  `engine` has PegaEngine's methods; `version` is what clients must announce."""

    def __init__(self, engine, *, version: str = R.PROTOCOL_VERSION, registry: Optional[TensorRegistry] = None):
        self.engine = engine
        self.version = version
        self.registry = registry or TensorRegistry()
        self.sessions = SessionRegistry()
        self.shutdown_requested = threading.Event()
        self._instances_lock = threading.Lock()
        self._instances: Dict[str, None] = {}       # registered instance ids, in registration order

    # ---- helpers
    @staticmethod
    def _ok():
        return pb.ResponseStatus(ok=True, message="")

    def _engine_call(self, context, fn):
        try:
            return fn()
        except Exception as e:       # engine errors carry their variant in `.kind`
            context.abort(_status_of(e), str(e))

    def cleanup_instance(self, instance_id: str) -> int:
        """service.rs:59-82: drop the instance's mapped tensors, then the instance (a missing instance is fine)."""
        removed = self.registry.drop_instance(instance_id)
        with self._instances_lock:
            self._instances.pop(instance_id, None)
        try:
            self.engine.unregister_instance(instance_id)
        except Exception:
            pass
        return removed

    def instance_ids(self) -> List[str]:
        """The engine's registered instances (lib.rs:477-484); an engine without that call is
        represented by what this service registered itself."""
        lister = getattr(self.engine, "list_instance_ids", None)
        if lister is not None:
            return list(lister())
        with self._instances_lock:
            return list(self._instances)

    # ---- RPCs
    def RegisterContextBatch(self, req, context):
        if req.client_version != self.version:
            context.abort(grpc.StatusCode.FAILED_PRECONDITION,
                          f"PegaFlow version mismatch: client={req.client_version or '<missing>'} server={self.version}")
        if req.device_id < 0:
            context.abort(grpc.StatusCode.INVALID_ARGUMENT, f"device_id {req.device_id} must be >= 0")
        if req.tp_size == 0:
            context.abort(grpc.StatusCode.INVALID_ARGUMENT, "tp_size must be > 0")
        if req.world_size == 0:
            context.abort(grpc.StatusCode.INVALID_ARGUMENT, "world_size must be > 0")
        if req.tp_rank >= req.tp_size:
            context.abort(grpc.StatusCode.INVALID_ARGUMENT, f"tp_rank {req.tp_rank} out of range (tp_size {req.tp_size})")
        n = len(req.layer_names)
        if n == 0 or any(len(x) != n for x in (req.wrapper_bytes, req.num_blocks, req.bytes_per_block,
                                               req.kv_stride_bytes, req.segments)):
            context.abort(grpc.StatusCode.INVALID_ARGUMENT,
                          f"all layer arrays must have the same non-zero length (got layer_names={n})")
        key = f"{req.instance_id}:tp{req.tp_rank}:pp{req.pp_rank}:dev{req.device_id}"
        try:
            regions = self.registry.register_layers(key, req.device_id, list(req.wrapper_bytes))
        except Exception as e:
            context.abort(grpc.StatusCode.INTERNAL, f"register tensor failed: {e}")
        try:
            self.engine.register_context_layer_batch_strided(
                req.instance_id, req.namespace, req.device_id, req.tp_rank, req.pp_rank, req.tp_size, req.world_size,
                list(req.layer_names), [r[0] for r in regions], [r[1] for r in regions], list(req.num_blocks),
                list(req.bytes_per_block), list(req.kv_stride_bytes), list(req.segments), None,
                list(req.layer_group_ids) if req.layer_group_ids else None,
                R.TRANSFER_MODE_NAME.get(req.transfer_mode, "direct"), req.page_first)
        except Exception as e:
            self.registry.drop_context(key)      # service.rs:318-330
            context.abort(_status_of(e), str(e))
        with self._instances_lock:
            self._instances[req.instance_id] = None
        return pb.RegisterContextResponse(status=self._ok())

    def Save(self, req, context):
        if req.device_id < 0:
            context.abort(grpc.StatusCode.INVALID_ARGUMENT, f"device_id {req.device_id} must be >= 0")
        for layer in req.saves:
            if len(layer.block_ids) != len(layer.block_hashes):
                context.abort(grpc.StatusCode.INVALID_ARGUMENT,
                              f"block_ids length {len(layer.block_ids)} does not match block_hashes "
                              f"{len(layer.block_hashes)} for layer {layer.layer_name}")
        saves = [(s.layer_name, list(s.block_ids), list(s.block_hashes)) for s in req.saves]
        self._engine_call(context, lambda: self.engine.batch_save(req.instance_id, req.tp_rank, req.pp_rank,
                                                                  req.device_id, saves))
        return pb.SaveResponse(status=self._ok())

    def Load(self, req, context):
        if req.device_id < 0:
            context.abort(grpc.StatusCode.INVALID_ARGUMENT, f"device_id {req.device_id} must be >= 0")
        groups = [list(g.layer_names) for g in req.groups]
        loads = []
        for load in req.loads:
            if len(load.lease) != 16:
                context.abort(grpc.StatusCode.INVALID_ARGUMENT, f"query lease must be 16 bytes, got {len(load.lease)}")
            loads.append((bytes(load.lease),
                          [[t.block_id if t.WhichOneof("target") else None for t in ids.targets]
                           for ids in load.block_ids_by_group]))
        self._engine_call(context, lambda: self.engine.batch_load_shm(req.instance_id, req.tp_rank, req.device_id,
                                                                      req.load_state_shm, groups, loads))
        return pb.LoadResponse(status=self._ok())

    def QueryPrefetch(self, req, context):
        if not req.req_id:
            context.abort(grpc.StatusCode.INVALID_ARGUMENT, "req_id must not be empty")
        hashes = list(req.block_hashes)

        def run():
            if req.group_id == 0:
                blocks, _missing = self.engine.query_prefix(req.instance_id, hashes, req.req_id)
                positions = list(range(len(blocks)))
            else:
                found = self.engine.query_group_membership(req.instance_id, req.group_id, hashes)
                positions = [i for i, b in enumerate(found) if b is not None]
                blocks = [found[i] for i in positions]
            if not len(blocks):
                return pb.QueryReady(num_hit_blocks=0, lease=b"")
            lease = self.engine.create_query_lease(req.instance_id, blocks)
            return pb.QueryReady(num_hit_blocks=len(blocks), lease=lease,
                                 hit_positions=positions if req.group_id else [])

        return pb.QueryResponse(ready=self._engine_call(context, run))

    def Release(self, req, context):
        if req.lease:
            self._engine_call(context, lambda: self.engine.release_query_lease(bytes(req.lease)))
        return pb.ReleaseResponse()

    def UnregisterContext(self, req, context):
        self.registry.drop_instance(req.instance_id)
        self._engine_call(context, lambda: self.engine.unregister_instance(req.instance_id))
        return pb.UnregisterResponse(status=self._ok())

    def Health(self, req, context):
        return pb.HealthResponse(status=self._ok())

    def Shutdown(self, req, context):
        self.shutdown_requested.set()
        return pb.ShutdownResponse(status=self._ok())

    def Session(self, req, context):
        if not req.instance_id:
            context.abort(grpc.StatusCode.INVALID_ARGUMENT, "instance_id must not be empty")
        token = self.sessions.install(req.instance_id, req.namespace, req.tp_size, req.world_size)
        closed = threading.Event()
        context.add_callback(closed.set)          # the client went away, or the server is stopping
        # No events are defined yet: the stream just stays open.
        while not closed.wait(0.2):
            if not context.is_active():
                break
        if self.sessions.take(req.instance_id, token):
            self.cleanup_instance(req.instance_id)
        return
        yield  # pragma: no cover  (makes this a generator: a server-streaming handler)

    def _unimplemented(self, req, context):
        context.abort(grpc.StatusCode.UNIMPLEMENTED, "cross-node transfer is not part of this library")


def _handlers(service: EngineService):
    table = {}
    for name, (req, resp, streaming) in R.METHODS.items():
        fn = getattr(service, name, service._unimplemented)
        make = grpc.unary_stream_rpc_method_handler if streaming else grpc.unary_unary_rpc_method_handler
        table[name] = make(fn, request_deserializer=R.message_class(req).FromString,
                           response_serializer=R.message_class(resp).SerializeToString)
    return grpc.method_handlers_generic_handler(R.SERVICE, table)


class EngineServer:
    def __init__(self, service: EngineService, server: grpc.Server, port: int):
        self.service, self._server, self.port = service, server, port

    def stop(self, grace: float = 1.0):
        self._server.stop(grace).wait()

    def wait_for_shutdown_request(self, timeout: Optional[float] = None) -> bool:
        return self.service.shutdown_requested.wait(timeout)


def serve(engine, address: str = "127.0.0.1:0", *, version: str = R.PROTOCOL_VERSION, max_workers: int = 16,
          registry: Optional[TensorRegistry] = None) -> EngineServer:
    """Start the sidecar on `address` ("host:port", port 0 = any free port) and return at once."""
    service = EngineService(engine, version=version, registry=registry)
    server = grpc.server(futures.ThreadPoolExecutor(max_workers=max_workers, thread_name_prefix="pf-rpc"),
                         options=[("grpc.max_receive_message_length", MAX_MESSAGE_BYTES),
                                  ("grpc.max_send_message_length", MAX_MESSAGE_BYTES)])
    server.add_generic_rpc_handlers((_handlers(service),))
    port = server.add_insecure_port(address)
    if port == 0:
        raise RuntimeError(f"could not bind {address}")
    server.start()
    return EngineServer(service, server, port)


def prometheus_text(metrics: dict) -> str:
    """The engine's transfer and pool counters in the Prometheus text format, under the reference's
    instrument names (pegaflow-core/src/metrics.rs:229-241,325-349).  Its two duration histograms are
    given as their sum and count; counters carry the `_total` suffix the exposition format asks for."""
    rows = [
        ("pegaflow_save_bytes_total", "counter", "Total bytes saved from GPU to CPU storage", metrics["save_bytes"]),
        ("pegaflow_save_duration_sum", "untyped", "Save operation latency in seconds (sum)", metrics["save_duration_seconds"]),
        ("pegaflow_save_duration_count", "untyped", "Save operations", metrics["save_batches"]),
        ("pegaflow_load_bytes_total", "counter", "Total bytes loaded from CPU storage to GPU", metrics["load_bytes"]),
        ("pegaflow_load_duration_sum", "untyped", "Load operation latency in seconds (sum)", metrics["load_duration_seconds"]),
        ("pegaflow_load_duration_count", "untyped", "Load operations", metrics["load_tasks"]),
        ("pegaflow_load_failures_total", "counter", "Load operation failures (e.g., transfer errors)", metrics["load_failures"]),
        ("pegaflow_pool_capacity_bytes", "gauge", "Pinned pool capacity", metrics["pool_capacity_bytes"]),
        ("pegaflow_pool_used_bytes", "gauge", "Pinned pool bytes in use", metrics["pool_used_bytes"]),
        ("pegaflow_pool_alloc_failures_total", "counter", "Pinned pool allocation failures", metrics["pool_alloc_failures"]),
    ]
    out = []
    for name, kind, text, value in rows:
        out += [f"# HELP {name} {text}", f"# TYPE {name} {kind}", f"{name} {value}"]
    return "\n".join(out) + "\n"


class InflightSweeper:
    """pegaflow-server/src/lib.rs:612-648: every `interval` seconds drop the blocks that have been waiting longer
    than `max_age` for slots that never came (a rank or a layer that did not save).  The reference's constants:
    60 s and 300 s."""

    def __init__(self, engine, interval: float = 60.0, max_age: float = 300.0):
        self.engine, self.interval, self.max_age = engine, interval, max_age
        self.cleaned = 0
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, name="pf-inflight-gc", daemon=True)
        self._thread.start()

    def _run(self):
        while not self._stop.wait(self.interval):
            try:
                self.cleaned += int(self.engine.gc_stale_inflight(self.max_age))
            except Exception:
                pass            # the engine is going away; the next tick finds the stop flag

    def stop(self):
        self._stop.set()
        self._thread.join(2.0)


class HttpEndpoints:
    """pegaflow-server/src/http_server.rs:22-196: `GET /health`, `GET /metrics` (when enabled),
    `GET /instances`, `POST /instances/cleanup[?id=<instance_id>]`, `POST /cache/memory/cleanup`, on a thread of
    their own."""

    def __init__(self, service: EngineService, address: str = "127.0.0.1:0", enable_prometheus: bool = True):
        import json
        from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
        from urllib.parse import parse_qs, urlsplit

        class Handler(BaseHTTPRequestHandler):
            def _send(self, code, body, kind="text/plain; charset=utf-8"):
                data = body.encode()
                self.send_response(code)
                self.send_header("Content-Type", kind)
                self.send_header("Content-Length", str(len(data)))
                self.end_headers()
                self.wfile.write(data)

            def _json(self, code, obj):
                self._send(code, json.dumps(obj), "application/json")

            def do_GET(self):
                path = urlsplit(self.path).path
                if path == "/health":
                    self._send(200, "ok")
                elif path == "/metrics" and enable_prometheus:
                    try:
                        self._send(200, prometheus_text(service.engine.metrics()), "text/plain; version=0.0.4")
                    except Exception as e:
                        self._send(200, f"# Error encoding metrics: {e}\n")
                elif path == "/instances":
                    self._json(200, {"instances": service.instance_ids()})
                else:
                    self._send(404, "metrics not enabled" if path == "/metrics" else "not found")

            def do_POST(self):
                url = urlsplit(self.path)
                if url.path == "/cache/memory/cleanup":
                    try:
                        self._json(200, service.engine.cleanup_memory_cache())
                    except Exception as e:
                        self._send(500, str(e))
                    return
                if url.path != "/instances/cleanup":
                    self._send(404, "not found")
                    return
                wanted = parse_qs(url.query).get("id")
                if wanted is None:        # every instance and every mapped tensor
                    ids = service.instance_ids()
                    tensors = sum(service.cleanup_instance(i) for i in ids)
                    self._json(200, {"removed_instances": ids, "removed_tensors": tensors})
                    return
                instance_id = wanted[0]
                known = instance_id in service.instance_ids()
                tensors = service.cleanup_instance(instance_id)
                if known or tensors > 0:
                    self._json(200, {"removed_instances": [instance_id], "removed_tensors": tensors})
                else:
                    self._send(404, f"instance {instance_id} not found")

            def log_message(self, fmt, *args):     # quiet: requests are not logged to stderr
                pass

        host, _, port = address.rpartition(":")
        self._httpd = ThreadingHTTPServer((host or "127.0.0.1", int(port)), Handler)
        self._httpd.daemon_threads = True
        self.port = self._httpd.server_address[1]
        self._thread = threading.Thread(target=self._httpd.serve_forever, name="pf-http", daemon=True)
        self._thread.start()

    def stop(self):
        self._httpd.shutdown()
        self._httpd.server_close()
        self._thread.join(2.0)


def main(argv=None):
    """``python -m pegaflow_b200.server --addr 127.0.0.1:50055 --pool-size 32gb`` (pegaflow-server's flags
    of the same names)."""
    import argparse

    from . import PegaEngine

    ap = argparse.ArgumentParser()
    ap.add_argument("--addr", default="127.0.0.1:50055")
    ap.add_argument("--pool-size", default="30gb")
    ap.add_argument("--use-hugepages", action="store_true")
    ap.add_argument("--http-addr", default="0.0.0.0:9091", help="health check, metrics and instance management")
    ap.add_argument("--enable-prometheus", default="true", choices=["true", "false"])
    args = ap.parse_args(argv)
    units = {"kb": 1 << 10, "mb": 1 << 20, "gb": 1 << 30, "tb": 1 << 40}
    text = args.pool_size.lower()
    pool = int(float(text[:-2]) * units[text[-2:]]) if text[-2:] in units else int(text)
    engine = PegaEngine(pool, args.use_hugepages)
    server = serve(engine, args.addr)
    http = HttpEndpoints(server.service, args.http_addr, args.enable_prometheus == "true")
    sweeper = InflightSweeper(engine)
    print(f"pegaflow_b200 engine server listening on port {server.port}", flush=True)
    print(f"pegaflow_b200 HTTP endpoints on port {http.port}", flush=True)
    try:
        server.wait_for_shutdown_request()
    except KeyboardInterrupt:
        pass
    sweeper.stop()
    http.stop()
    server.stop()
    engine.close()


if __name__ == "__main__":
    main()
