"""Generate ``scheduler_traces.json`` by driving the reference's own ``SchedulerConnector``.

Run where the reference checkout is available (``PEGAFLOW_REFERENCE``, default: a ``reference``
directory beside this repository).  The reference's scheduler-side connector
(python/pegaflow/connector/scheduler.py) is imported with its native extension stubbed out by the
reference's own ``unit_stubs`` helper and driven through scripted request lifecycles against fake
engine clients; what it answers at every step (matched tokens, load intents, save intents, leases
it releases) is recorded.  The scripts live in ``tests/scheduler_scripts.py`` so that the test can
replay exactly the same operations on this repository's ``SchedulerConnector``.  The output is
committed; the tests never need the reference at run time.
"""
import json
import os
import sys
from types import SimpleNamespace
from unittest.mock import MagicMock

_REPO = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
REF = os.environ.get("PEGAFLOW_REFERENCE", os.path.join(os.path.dirname(_REPO), "reference"))
sys.path.insert(0, os.path.join(REF, "python"))
from tests.unit_stubs import install_connector_unit_stubs  # noqa: E402  (the reference's tests package)

install_connector_unit_stubs()
from pegaflow.connector.common import ConnectorContext, PegaConnectorMode  # noqa: E402
from pegaflow.connector.scheduler import SchedulerConnector  # noqa: E402
from pegaflow.pegaflow import QueryLoading, QueryReady  # noqa: E402

import importlib.util  # noqa: E402

_spec = importlib.util.spec_from_file_location("scheduler_scripts", os.path.join(_REPO, "tests", "scheduler_scripts.py"))
scripts = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(scripts)


def make_reference_connector(clients, *, block_size, read_enabled, wait_for_full_prefix, group_count, recurrent_groups=0):
    ctx = ConnectorContext(
        instance_id="inst", namespace="ns", block_size=block_size, tp_size=1, world_size=1, tp_rank=None, device_id=None,
        engine_client=clients[0], state_manager=MagicMock(),
        mode=PegaConnectorMode.READ_WRITE if read_enabled else next(m for m in PegaConnectorMode
                                                                    if m is not PegaConnectorMode.READ_WRITE),
        wait_for_full_prefix=wait_for_full_prefix,
        tp_shards=None if len(clients) == 1 else SimpleNamespace(shard_count=len(clients)))
    kv_cache_config = None
    conn = SchedulerConnector(ctx, engine_clients=tuple(clients), kv_cache_config=kv_cache_config)
    if recurrent_groups:
        # one attention group followed by the recurrent-state groups, storage groups 1..n
        from pegaflow.connector.common import CacheGroupLayout

        names = (("attn",),) + tuple((f"mamba{g}",) for g in range(1, recurrent_groups + 1))
        conn._cache_groups = CacheGroupLayout(
            layer_names=names, hash_group_index=0, has_recurrent_state=True,
            recurrent_group_indices=frozenset(range(1, recurrent_groups + 1)),
            recurrent_layer_names=frozenset(n for g in names[1:] for n in g),
            storage_group_ids=tuple(range(recurrent_groups + 1)))
    if group_count != 1:
        # attention-only groups that share the hash cadence: the layout only needs the group count
        object.__setattr__(conn._cache_groups, "layer_names", tuple(() for _ in range(group_count)))
    return conn


def main():
    out = {}
    for name, script in scripts.SCRIPTS.items():
        out[name] = scripts.run_script(script, make_reference_connector, QueryReady, QueryLoading)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "scheduler_traces.json")
    with open(path, "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
    print(path, {k: len(v) for k, v in out.items()})


if __name__ == "__main__":
    main()
