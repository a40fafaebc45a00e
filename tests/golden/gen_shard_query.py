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


if __name__ == "__main__":
    out = cases.run_all(Adapter, QueryReady, QueryLoading)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "shard_query.json")
    with open(path, "w") as f:
        json.dump(out, f, sort_keys=True)
        f.write("\n")
    kinds = {}
    for r in out:
        key = (r["kind"], "ok" if "ok" in r["outcome"] else r["outcome"]["error"][0])
        kinds[key] = kinds.get(key, 0) + 1
    print(path, kinds)
