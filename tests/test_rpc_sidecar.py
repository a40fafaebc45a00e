"""The gRPC sidecar and its client on CPU: real wire (loopback), the oracle engine model behind the
service, numpy buffers standing in for mapped KV tensors.  Scenarios follow the reference's server
tests: pegaflow-server/tests/mock_vllm_rpc_e2e.rs:318-360 (TP=2: a query before both ranks saved
is a miss, then a hit, then a load per rank through a shared-memory LoadState), service.rs:1080-1188
(validation and status codes) and session.rs:82-105 (a newer session supersedes an older one)."""
import pickle
import time

import numpy as np
import pytest

grpc = pytest.importorskip("grpc")

from oracle.engine_model import OracleEngine  # noqa: E402
from pegaflow_b200 import PegaFlowError, PegaflowInternal, PyLoadState, rpc_proto  # noqa: E402
from pegaflow_b200.connector import QueryReady  # noqa: E402
from pegaflow_b200.rpc_client import EngineRpcClient  # noqa: E402
from pegaflow_b200.server import SessionRegistry, serve  # noqa: E402
from tests import scenarios as sc  # noqa: E402


class EngineUnderRpc(OracleEngine):
    """The oracle model with the two call shapes the service uses that it lacks: a request id on the
    prefix query, and a load that reports through a LoadState segment (lib.rs:654-680)."""

    def query_prefix(self, instance_id, hashes, req_id=""):
        return super().query_prefix(instance_id, hashes)

    def batch_load_shm(self, instance_id, tp_rank, device_id, shm_name, layer_groups, loads):
        state = PyLoadState(attach_to=shm_name)      # must be attachable before anything else happens
        try:
            self.batch_load(instance_id, tp_rank, device_id, layer_groups, loads)
        except Exception:
            state.set_error()
            raise
        state.set_completed()


class NumpyRegistry:
    """Wrapper bytes are a pickled index into buffers this test owns."""

    def __init__(self, buffers):
        self.buffers, self.contexts = buffers, {}

    def register_layers(self, key, device_id, wrapper_bytes):
        idx = [pickle.loads(b) for b in wrapper_bytes]
        if any(i not in self.buffers for i in idx):
            raise RuntimeError("unknown tensor")
        self.contexts.setdefault(key, []).extend(idx)
        return [(self.buffers[i].ctypes.data, self.buffers[i].nbytes) for i in idx]

    def drop_context(self, key):
        return len(self.contexts.pop(key, []))

    def drop_instance(self, instance_id):
        keys = [k for k in self.contexts if k.startswith(instance_id + ":")]
        return sum(len(self.contexts.pop(k)) for k in keys)


@pytest.fixture
def sidecar():
    buffers = {}
    engine = EngineUnderRpc(16 << 20)
    registry = NumpyRegistry(buffers)
    server = serve(engine, "127.0.0.1:0", registry=registry)
    client = EngineRpcClient(f"http://127.0.0.1:{server.port}", timeout=20)
    yield engine, registry, buffers, server, client
    client.close()
    server.stop(0.2)


def _register(client, buffers, instance, rank, layers, n_blocks=8, seg=1024, tp_size=2, world=2, version=None):
    names = [f"model.layers.{i}.attn" for i in range(layers)]
    keys = []
    for i in range(layers):
        key = (instance, rank, i)
        buffers[key] = sc.seeded_bytes(n_blocks * seg, 50 + 10 * rank + i)
        keys.append(pickle.dumps(key))
    c = client if version is None else EngineRpcClient(client.endpoint(), timeout=20, client_version=version)
    return names, c.register_context_batch(instance, "ns", rank, 0, tp_size, world, rank, names, keys, [n_blocks] * layers,
                                           [seg] * layers, [0] * layers, [1] * layers, "direct", False)


def test_tp2_miss_then_hit_then_load_per_rank_over_the_wire(sidecar):
    engine, registry, buffers, server, client = sidecar
    assert client.health() == (True, "")
    names, reply = _register(client, buffers, "tp", 0, 2)
    assert reply == (True, "")
    _, reply = _register(client, buffers, "tp", 1, 2)
    assert reply == (True, "")
    before = {k: v.copy() for k, v in buffers.items()}
    h = sc.make_block_hashes(3, 9)
    assert client.save("tp", 0, 0, 0, [(n, [1, 2, 3], h) for n in names]) == (True, "")
    q = client.query_prefetch("tp", h, "req-1")
    assert isinstance(q, QueryReady) and (q.num_hit_blocks, q.lease, q.hit_positions) == (0, b"", [])
    assert client.save("tp", 1, 0, 1, [(n, [4, 5, 6], h) for n in names]) == (True, "")
    q = client.query_prefetch("tp", h, "req-1")
    assert q.num_hit_blocks == 3 and len(q.lease) == 16 and q.hit_positions == []
    for rank, dst in ((0, [5, 6, 7]), (1, [0, None, 2])):       # None: a position without a destination
        for i in range(2):
            buffers[("tp", rank, i)][:] = 0
        state = PyLoadState()
        assert client.load("tp", rank, rank, state.shm_name(), [names], [(q.lease, [dst])]) == (True, "")
        deadline = time.time() + 10
        while not state.is_ready() and time.time() < deadline:
            time.sleep(0.01)
        assert state.get_state() == 1
        src = [1, 2, 3] if rank == 0 else [4, 5, 6]
        for i in range(2):
            want = np.zeros_like(before[("tp", rank, i)]).reshape(8, 1024)
            for s, d in zip(src, dst):
                if d is not None:
                    want[d] = before[("tp", rank, i)].reshape(8, 1024)[s]
            assert np.array_equal(buffers[("tp", rank, i)].reshape(8, 1024), want)
    # both ranks consumed the lease: releasing it again is harmless, loading with it is not possible
    client.release(q.lease)
    state = PyLoadState()
    with pytest.raises(PegaflowInternal, match="unknown or expired"):
        client.load("tp", 0, 0, state.shm_name(), [names], [(q.lease, [[1, 2, 3]])])
    assert state.get_state() == -1
    assert client.unregister_context("tp") == (True, "") and registry.contexts == {}
    with pytest.raises(PegaFlowError, match="FAILED_PRECONDITION.*instance tp not found"):
        client.query_prefetch("tp", h, "req-2")


def test_validation_and_status_codes(sidecar):
    engine, registry, buffers, server, client = sidecar
    with pytest.raises(PegaFlowError, match="FAILED_PRECONDITION.*version mismatch: client=0.0.1 server=" +
                       rpc_proto.PROTOCOL_VERSION):
        _register(client, buffers, "v", 0, 1, version="0.0.1")
    with pytest.raises(PegaFlowError, match="client=<missing>"):
        _register(client, buffers, "v", 0, 1, version="")
    with pytest.raises(ValueError, match="tp_rank 3 out of range \\(tp_size 2\\)"):
        _register(client, buffers, "v", 3, 1)
    with pytest.raises(ValueError, match="tp_size must be > 0"):
        _register(client, buffers, "v", 0, 1, tp_size=0)
    with pytest.raises(ValueError, match="same non-zero length"):
        client.register_context_batch("v", "ns", 0, 0, 1, 1, 0, ["a", "b"], [b"x"], [1, 1], [1, 1], [0, 0], [1, 1], "direct", False)
    with pytest.raises(ValueError, match="unknown transfer_backend"):
        client.register_context_batch("v", "ns", 0, 0, 1, 1, 0, ["a"], [b"x"], [1], [1], [0], [1], "dma", False)
    with pytest.raises(PegaflowInternal, match="register tensor failed"):
        client.register_context_batch("v", "ns", 0, 0, 1, 1, 0, ["a"], [pickle.dumps("nope")], [1], [1], [0], [1], "direct", False)
    # a registration the engine refuses unmaps what the server had mapped for it (service.rs:318-330)
    buffers["small"] = np.zeros(1024, dtype=np.uint8)
    with pytest.raises(ValueError, match="too small"):
        client.register_context_batch("v", "ns", 0, 0, 1, 1, 0, ["a"], [pickle.dumps("small")], [8], [1024], [0], [1], "direct", False)
    assert registry.contexts == {}
    names, reply = _register(client, buffers, "v", 0, 1, tp_size=1, world=1)
    assert reply == (True, "")
    with pytest.raises(ValueError, match="does not match block_hashes"):
        client.save("v", 0, 0, 0, [(names[0], [1, 2], [b"h"])])
    with pytest.raises(ValueError, match="device_id -1 must be >= 0"):
        client.save("v", 0, 0, -1, [])
    with pytest.raises(ValueError, match="req_id must not be empty"):
        client.query_prefetch("v", [b"h"], "")
    with pytest.raises(PegaFlowError, match="FAILED_PRECONDITION.*device 4 not found"):
        client.save("v", 0, 0, 4, [(names[0], [1], [b"h"])])
    with pytest.raises(ValueError, match="16 bytes"):
        client.load("v", 0, 0, "x", [names], [(b"short", [[1]])])
    with pytest.raises(PegaFlowError, match="UNIMPLEMENTED"):
        client._call("RdmaHandshake", rpc_proto.pb.RdmaHandshakeRequest(requester_id="peer"))
    assert client.shutdown() == (True, "") and server.wait_for_shutdown_request(1.0)


def test_unreachable_server_is_a_zero_hit_query_not_an_error():
    client = EngineRpcClient("http://127.0.0.1:1", timeout=0.5)       # nobody listens there (lib.rs:505-519)
    q = client.query_prefetch("inst", [b"h"], "req")
    assert (q.num_hit_blocks, q.lease) == (0, b"")
    with pytest.raises(PegaFlowError):
        client.health()
    client.close()


def test_session_end_cleans_the_instance_up_unless_superseded(sidecar):
    engine, registry, buffers, server, client = sidecar
    names, reply = _register(client, buffers, "live", 0, 1, tp_size=1, world=1)
    assert reply == (True, "") and len(registry.contexts) == 1
    with pytest.raises(ValueError):
        client.start_session_watcher("", "ns", 1, 1)
    first = EngineRpcClient(client.endpoint(), timeout=20)
    first.start_session_watcher("live", "ns", 1, 1)
    deadline = time.time() + 5
    while server.service.sessions.topology("live") is None and time.time() < deadline:
        time.sleep(0.01)
    second = EngineRpcClient(client.endpoint(), timeout=20)
    second.start_session_watcher("live", "ns2", 1, 1)                  # e.g. the worker restarted and reconnected
    while server.service.sessions.topology("live") != ("ns2", 1, 1) and time.time() < deadline:
        time.sleep(0.01)
    first.close()                                                      # the old stream ends: superseded, no cleanup
    time.sleep(0.6)
    assert client.query_prefetch("live", [b"h"], "r").num_hit_blocks == 0 and len(registry.contexts) == 1
    second.close()                                                     # the live stream ends: the instance goes
    deadline = time.time() + 5
    while registry.contexts and time.time() < deadline:
        time.sleep(0.05)
    assert registry.contexts == {}
    with pytest.raises(PegaFlowError, match="instance live not found"):
        client.query_prefetch("live", [b"h"], "r")


def test_session_registry_tokens():
    reg = SessionRegistry()                                            # session.rs:86-104
    first = reg.install("inst", "ns1", 8, 8)
    second = reg.install("inst", "ns2", 4, 4)
    assert first != second and reg.topology("inst") == ("ns2", 4, 4)
    assert not reg.take("inst", first)
    assert reg.take("inst", second) and reg.topology("inst") is None


def test_wire_contract_field_numbers():
    """Spot checks against pegaflow-proto/proto/engine.proto: encoded bytes, not Python attribute names."""
    pb = rpc_proto.pb
    assert pb.SaveRequest(instance_id="i", pp_rank=3).SerializeToString() == b"\x0a\x01i\x28\x03"            # 1, 5
    assert pb.RegisterContextRequest(page_first=True, transfer_mode=1).SerializeToString() == b"\x88\x01\x01\x90\x01\x01"  # 17, 18
    assert pb.LoadBlockTarget(block_id=0).SerializeToString() == b"\x08\x00" and pb.LoadBlockTarget().SerializeToString() == b""
    assert pb.QueryResponse(loading=pb.QueryLoading()).SerializeToString() == b"\x0a\x00"
    assert pb.QueryReady(num_hit_blocks=2, lease=b"ab", hit_positions=[1, 5]).SerializeToString() == b"\x08\x02\x12\x02ab\x1a\x02\x01\x05"
    assert rpc_proto.method_path("QueryPrefetch") == "/pegaflow.Engine/QueryPrefetch"


def test_http_health_metrics_and_instance_management(sidecar):
    """pegaflow-server/src/http_server.rs:22-196: /health, /metrics, /instances, /instances/cleanup[?id=]."""
    import json
    import urllib.error
    import urllib.request

    from pegaflow_b200.server import HttpEndpoints, prometheus_text

    engine, registry, buffers, server, client = sidecar
    counters = dict(save_bytes=4096, save_duration_seconds=0.5, save_batches=2, load_bytes=1024,
                    load_duration_seconds=0.25, load_tasks=1, load_failures=0, pool_capacity_bytes=16 << 20,
                    pool_used_bytes=8192, pool_alloc_failures=3)
    engine.metrics = lambda: counters
    http = HttpEndpoints(server.service, "127.0.0.1:0")
    base = f"http://127.0.0.1:{http.port}"

    def get(path):
        with urllib.request.urlopen(base + path, timeout=10) as r:
            return r.status, r.read().decode()

    def post(path):
        try:
            with urllib.request.urlopen(urllib.request.Request(base + path, data=b"", method="POST"), timeout=10) as r:
                return r.status, r.read().decode()
        except urllib.error.HTTPError as e:
            return e.code, e.read().decode()

    try:
        assert get("/health") == (200, "ok")
        assert json.loads(get("/instances")[1]) == {"instances": []}
        _register(client, buffers, "a", 0, 2, tp_size=1, world=1)
        _register(client, buffers, "b", 0, 3, tp_size=1, world=1)
        assert json.loads(get("/instances")[1]) == {"instances": ["a", "b"]}
        code, text = get("/metrics")
        assert code == 200 and text == prometheus_text(counters)
        for line in ("pegaflow_save_bytes_total 4096", "pegaflow_load_bytes_total 1024", "pegaflow_load_failures_total 0",
                     "pegaflow_save_duration_sum 0.5", "pegaflow_load_duration_count 1",
                     "pegaflow_pool_used_bytes 8192", "pegaflow_pool_alloc_failures_total 3"):
            assert line in text.splitlines()
        assert post("/instances/cleanup?id=nobody")[0] == 404
        assert json.loads(post("/instances/cleanup?id=a")[1]) == {"removed_instances": ["a"], "removed_tensors": 2}
        assert json.loads(get("/instances")[1]) == {"instances": ["b"]}
        assert json.loads(post("/instances/cleanup")[1]) == {"removed_instances": ["b"], "removed_tensors": 3}
        assert json.loads(get("/instances")[1]) == {"instances": []} and registry.contexts == {}
        engine.cleanup_memory_cache = lambda: {"evicted_blocks": 3, "evicted_bytes": 6144, "reclaimed_bytes": 4096,
                                               "still_referenced_blocks": 1}
        assert json.loads(post("/cache/memory/cleanup")[1]) == {"evicted_blocks": 3, "evicted_bytes": 6144,
                                                                "reclaimed_bytes": 4096, "still_referenced_blocks": 1}
        with pytest.raises(urllib.error.HTTPError):
            get("/nothing")
    finally:
        http.stop()
    quiet = HttpEndpoints(server.service, "127.0.0.1:0", enable_prometheus=False)
    try:
        with pytest.raises(urllib.error.HTTPError) as e:
            urllib.request.urlopen(f"http://127.0.0.1:{quiet.port}/metrics", timeout=10)
        assert e.value.code == 404 and e.value.read() == b"metrics not enabled"
    finally:
        quiet.stop()


def test_rpc_client_surface_matches_the_reference_stub():
    """python/pegaflow/pegaflow.pyi through tests/golden/engine_client_surface.json: every method of the reference's
    EngineRpcClient exists here with the same parameters in the same order, the constructor included."""
    import inspect
    import json
    import os

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = json.load(open(os.path.join(root, "tests", "golden", "engine_client_surface.json")))["classes"]["EngineRpcClient"]
    for method, params in spec["methods"].items():
        assert hasattr(EngineRpcClient, method), f"EngineRpcClient.{method} is missing"
        sig = inspect.signature(getattr(EngineRpcClient, method))
        got = [(p.name, p.default is not inspect.Parameter.empty) for p in sig.parameters.values()
               if p.name != "self" and p.kind not in (p.VAR_POSITIONAL, p.VAR_KEYWORD, p.KEYWORD_ONLY)]
        want = [tuple(x) for x in params]
        assert got[:len(want)] == want, f"EngineRpcClient.{method}: {got} != {want}"
        assert all(has_default for _, has_default in got[len(want):]), f"{method}: extra parameters must be optional"


def test_inflight_sweeper_calls_the_engine_until_stopped():
    """pegaflow-server/src/lib.rs:612-648: a background sweep with the maximum age it was given."""
    from pegaflow_b200.server import InflightSweeper

    class Engine:
        def __init__(self):
            self.ages = []

        def gc_stale_inflight(self, max_age):
            self.ages.append(max_age)
            return 2

    engine = Engine()
    sweeper = InflightSweeper(engine, interval=0.02, max_age=300.0)
    deadline = time.time() + 5
    while len(engine.ages) < 3 and time.time() < deadline:
        time.sleep(0.01)
    sweeper.stop()
    seen = len(engine.ages)
    assert seen >= 3 and set(engine.ages) == {300.0} and sweeper.cleaned == 2 * seen
    time.sleep(0.1)
    assert len(engine.ages) == seen, "the sweep went on after stop()"
