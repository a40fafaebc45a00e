"""Generate ``shard_query.json``: what the reference's TpShardQueryClient
(python/pegaflow/connector/tp_shards.py) answers, raises and releases in the scripted scenarios of
``tests/shard_query_cases.py``.  The reference is imported with its own ``unit_stubs`` in place of
the native extension.

    PEGAFLOW_REFERENCE=<checkout> python tests/golden/gen_shard_query.py
"""
import importlib.util
import json
import os
import sys

_REPO = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
REF = os.environ.get("PEGAFLOW_REFERENCE", os.path.join(os.path.dirname(_REPO), "reference"))
sys.path.insert(0, os.path.join(REF, "python"))
from tests.unit_stubs import install_connector_unit_stubs  # noqa: E402  (the reference's tests package)

install_connector_unit_stubs()
from pegaflow.connector.tp_shards import TpShardQueryClient  # noqa: E402
from pegaflow.pegaflow import QueryLoading, QueryReady  # noqa: E402

_spec = importlib.util.spec_from_file_location("shard_query_cases", os.path.join(_REPO, "tests", "shard_query_cases.py"))
cases = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(cases)


class Adapter:
    def __init__(self, shards):
        self.client = TpShardQueryClient(shards)

    def prefix(self, instance_id, hashes, req_id, wait):
        got = self.client.query(instance_id, hashes, req_id, wait)
        return None if got is None else [got.num_hit_blocks, [lease.decode() for lease in got.leases]]

    def membership(self, instance_id, hashes, req_id, group_id):
        return [[list(p), lease.decode()] for p, lease in self.client.query_group_membership(instance_id, hashes, req_id, group_id)]


def hybrid_adapter(shards, group_ids):
    """The reference's scheduler connector with a hybrid cache-group layout: one attention group and
    one recurrent group per id, driven through its own lookup entry point."""
    from unittest.mock import MagicMock

    from pegaflow.connector.common import CacheGroupLayout, ConnectorContext, PegaConnectorMode
    from pegaflow.connector.scheduler import SchedulerConnector

    ctx = ConnectorContext(
        instance_id="inst", namespace="ns", block_size=16, tp_size=1, world_size=1, tp_rank=None, device_id=None,
        engine_client=shards[0], state_manager=MagicMock(), mode=PegaConnectorMode.READ_WRITE, wait_for_full_prefix=False,
        tp_shards=None if len(shards) == 1 else type("T", (), {"shard_count": len(shards)})())
    conn = SchedulerConnector(ctx, engine_clients=tuple(shards), kv_cache_config=None)
    n = len(group_ids)
    conn._cache_groups = CacheGroupLayout(
        layer_names=(("attn",),) + tuple((f"mamba{g}",) for g in group_ids), hash_group_index=0, has_recurrent_state=True,
        recurrent_group_indices=frozenset(range(1, n + 1)), recurrent_layer_names=frozenset(f"mamba{g}" for g in group_ids),
        storage_group_ids=(0,) + tuple(group_ids))

    class H:
        def hybrid(self, instance_id, hashes, req_id, wait):
            got = conn._count_available_block_prefix(hashes, req_id)
            if got is None:
                return None
            hold = got.recurrent_hold
            return {"hit": got.num_hit_blocks, "leases": [x.decode() for x in got.leases],
                    "recurrent_leases": [[x.decode() for x in g] for g in hold.leases] if hold else [],
                    "recurrent_positions": [[list(p) for p in g] for g in hold.hit_positions] if hold else [],
                    "checkpoint": hold.checkpoint if hold else None, "usable": list(got.usable_positions)}
    return H()


if __name__ == "__main__":
    out = cases.run_all(Adapter, QueryReady, QueryLoading)
    out += cases.run_hybrid(hybrid_adapter, QueryReady, QueryLoading)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "shard_query.json")
    with open(path, "w") as f:
        json.dump(out, f, sort_keys=True)
        f.write("\n")
    kinds = {}
    for r in out:
        key = (r["kind"], "ok" if "ok" in r["outcome"] else r["outcome"]["error"][0])
        kinds[key] = kinds.get(key, 0) + 1
    print(path, kinds)
