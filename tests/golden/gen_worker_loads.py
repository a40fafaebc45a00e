"""Generate ``worker_loads.json``: the load requests the reference's WorkerConnector.start_load_kv
(python/pegaflow/connector/worker.py:549-710) sends to the engine for the hybrid load intents of
``tests/worker_load_cases.py``.  The reference is imported with its own ``unit_stubs`` in place of
the native extension; cache-group layouts are built from vLLM's spec classes.

    PEGAFLOW_REFERENCE=<checkout> python tests/golden/gen_worker_loads.py
"""
import importlib.util
import json
import os
import sys
from unittest.mock import MagicMock

_REPO = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
REF = os.environ.get("PEGAFLOW_REFERENCE", os.path.join(os.path.dirname(_REPO), "reference"))
sys.path.insert(0, os.path.join(REF, "python"))
from tests.unit_stubs import install_connector_unit_stubs  # noqa: E402  (the reference's tests package)

install_connector_unit_stubs()
from pegaflow.connector.common import (ConnectorContext, LoadIntent, PegaConnectorMetadata, PegaConnectorMode,  # noqa: E402
                                       RecurrentLoadHold, TpShardTopology)
from pegaflow.connector.worker import WorkerConnector  # noqa: E402

_spec = importlib.util.spec_from_file_location("worker_load_cases", os.path.join(_REPO, "tests", "worker_load_cases.py"))
cases = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(cases)


def start_load(layout, shard, shards, layers, intents, client):
    topology = None
    if shards > 1:
        topology = TpShardTopology.from_config("e0", [f"e{i}" for i in range(shards)], shards, shards)
    ctx = ConnectorContext(instance_id="inst", namespace="ns", block_size=16, tp_size=shards, world_size=shards,
                           tp_rank=shard, device_id=0, engine_client=client, state_manager=MagicMock(),
                           mode=PegaConnectorMode.READ_WRITE, tp_shards=topology)
    worker = WorkerConnector(ctx, kv_cache_config=cases.kv_cache_config(layout))
    try:
        worker._registered_layers = list(layers)
        meta = PegaConnectorMetadata(load_intents=cases.build_intents(intents, LoadIntent, RecurrentLoadHold))
        worker.start_load_kv(meta, None)
    finally:
        worker._save_queue.put(None)
        worker._save_thread.join()


if __name__ == "__main__":
    out = cases.run_all(start_load)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "worker_loads.json")
    with open(path, "w") as f:
        json.dump(out, f, sort_keys=True, indent=1)
        f.write("\n")
    print(path, {k: ("error" if "error" in v else len(v["calls"])) for k, v in out.items()})
