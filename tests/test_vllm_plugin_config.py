"""The vLLM plug-in's construction rules on CPU, with a stand-in for vLLM's config object: where the engine
lives (in the process, or behind the sidecar when `pegaflow.host` / `pegaflow.port` are given, as
python/pegaflow/connector/__init__.py:96-103 reads them), what each form refuses, and that the scheduler role
of the sidecar form opens the session's liveness stream (connector/__init__.py:200-211)."""
import os
import time
from types import SimpleNamespace

import pytest

pytest.importorskip("grpc")
pytest.importorskip("vllm")

from vllm.distributed.kv_transfer.kv_connector.v1.base import KVConnectorRole  # noqa: E402

from pegaflow_b200 import vllm_connector as plug  # noqa: E402
from pegaflow_b200.server import serve  # noqa: E402
from tests.test_rpc_sidecar import EngineUnderRpc, NumpyRegistry  # noqa: E402


def _config(extra, tp=1, pp=1, dp=1, engine_id="plug-test"):
    model = SimpleNamespace(model="tiny", dtype="bfloat16", use_mla=False, get_total_num_kv_heads=lambda: 2,
                            get_head_size=lambda: 64, get_total_num_hidden_layers=lambda: 4)
    return SimpleNamespace(
        kv_transfer_config=SimpleNamespace(engine_id=engine_id, get_from_extra_config=lambda k, d: extra.get(k, d)),
        instance_id="", cache_config=SimpleNamespace(block_size=16, cache_dtype="auto"), model_config=model,
        parallel_config=SimpleNamespace(tensor_parallel_size=tp, pipeline_parallel_size=pp, world_size=tp * pp,
                                        data_parallel_size=dp, data_parallel_rank_local=None),
        scheduler_config=SimpleNamespace(disable_hybrid_kv_cache_manager=True), additional_config={})


@pytest.fixture(autouse=True)
def _no_server_env(monkeypatch):
    monkeypatch.delenv("PEGAFLOW_HOST", raising=False)
    monkeypatch.delenv("PEGAFLOW_PORT", raising=False)


def test_in_process_form_refuses_more_than_one_worker():
    with pytest.raises(ValueError, match="2 workers: start the sidecar"):
        plug.PegaKVConnector(_config({}, tp=2), KVConnectorRole.SCHEDULER)
    with pytest.raises(ValueError, match="4 workers"):
        plug.PegaKVConnector(_config({}, tp=2, dp=2), KVConnectorRole.SCHEDULER)


def test_layerwise_hooks_cannot_be_combined_with_a_server():
    with pytest.raises(ValueError, match="pegaflow.layerwise needs the engine in the vLLM process"):
        plug.PegaKVConnector(_config({"pegaflow.port": 1, "pegaflow.layerwise": True}), KVConnectorRole.SCHEDULER)


def test_scheduler_role_of_the_sidecar_form_holds_the_session(monkeypatch):
    engine = EngineUnderRpc(1 << 20)
    server = serve(engine, "127.0.0.1:0", registry=NumpyRegistry({}))
    try:
        conn = plug.PegaKVConnector(_config({"pegaflow.port": server.port}, tp=2), KVConnectorRole.SCHEDULER)
        assert conn._remote and not conn._layerwise and conn._engine is None
        assert conn._client.endpoint() == f"http://127.0.0.1:{server.port}"
        deadline = time.time() + 10
        while server.service.sessions.topology("plug-test") is None and time.time() < deadline:
            time.sleep(0.02)
        namespace, tp_size, world_size = server.service.sessions.topology("plug-test")
        assert (tp_size, world_size) == (2, 2) and namespace == conn._namespace
        conn._client.close()
        # the environment wins over the extra config, as in the reference
        monkeypatch.setenv("PEGAFLOW_PORT", str(server.port))
        conn = plug.PegaKVConnector(_config({"pegaflow.port": 1, "pegaflow.host": "http://127.0.0.1"}),
                                    KVConnectorRole.SCHEDULER)
        assert conn._client.endpoint() == f"http://127.0.0.1:{server.port}" and conn._client.health() == (True, "")
        conn._client.close()
    finally:
        server.stop(0.2)


def test_global_device_id_undoes_cuda_visible_devices(monkeypatch):
    monkeypatch.delenv("CUDA_VISIBLE_DEVICES", raising=False)
    assert plug.global_device_id(3) == 3
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "4, 6")
    assert [plug.global_device_id(i) for i in range(3)] == [4, 6, 2]
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "GPU-3f2a,GPU-77aa")       # UUIDs cannot be mapped
    assert plug.global_device_id(1) == 1
