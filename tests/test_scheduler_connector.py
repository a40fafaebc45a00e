"""The scheduler-side connector against traces of the reference's own ``SchedulerConnector``
(python/pegaflow/connector/scheduler.py), recorded by ``tests/golden/gen_scheduler_traces.py``: the
same scripted request lifecycles are replayed here and every answer — matched tokens, load and save
intents, leases taken and given back — must be identical."""
import json
import os

import pytest

from tests import scheduler_scripts as scripts

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def golden():
    with open(os.path.join(HERE, "golden", "scheduler_traces.json")) as f:
        return json.load(f)


def _make(clients, *, block_size, read_enabled, wait_for_full_prefix, group_count):
    from pegaflow_b200.scheduler import SchedulerConnector

    assert group_count == 1
    return SchedulerConnector(clients, instance_id="inst", block_size=block_size, read_enabled=read_enabled,
                              wait_for_full_prefix=wait_for_full_prefix)


def test_every_script_has_a_trace(golden):
    assert sorted(golden) == sorted(scripts.SCRIPTS)


@pytest.mark.parametrize("name", sorted(scripts.SCRIPTS))
def test_replay_matches_the_reference(golden, name):
    from pegaflow_b200.connector import QueryLoading, QueryReady

    got = scripts.run_script(scripts.SCRIPTS[name], _make, QueryReady, QueryLoading)
    got = json.loads(json.dumps(got))       # tuples -> lists, like the stored trace
    want = golden[name]
    assert len(got) == len(want)
    for step, (g, w) in enumerate(zip(got, want)):
        assert g["op"] == w["op"], f"step {step}: the script changed after the trace was recorded"
        assert g["result"] == w["result"], f"step {step} {g['op']}: result differs"
        assert g["client_log"] == w["client_log"], f"step {step} {g['op']}: engine calls differ"
        assert g["live_leases"] == w["live_leases"], f"step {step} {g['op']}: leases held differ"


def test_scheduler_feeds_the_worker_connector_format():
    """The intents are what PegaWorkerConnector consumes: (request, lease, destination ids) for a load,
    (layer, ids, hashes) per registered layer for a save."""
    from pegaflow_b200.connector import QueryLoading, QueryReady
    from pegaflow_b200.scheduler import SchedulerConnector

    client = scripts.FakeClient("shard0", QueryReady, QueryLoading)
    client.store.update(scripts.H(i) for i in range(3))
    conn = SchedulerConnector([client], instance_id="inst", block_size=16)
    req = scripts.FakeRequest("q", range(4), 70)
    tokens, load_async = conn.get_num_new_matched_tokens(req, 0)
    assert (tokens, load_async) == (48, True)
    conn.update_state_after_alloc(req, scripts.FakeBlocks([3, 4, 5, 6, 7], 0), tokens)
    from types import SimpleNamespace as NS

    meta = conn.build_connector_meta(NS(
        scheduled_new_reqs=[NS(req_id="q", block_ids=([3, 4, 5, 6, 7],), num_computed_tokens=48)],
        scheduled_cached_reqs=NS(req_ids=[], new_block_ids=[], num_computed_tokens=[], resumed_req_ids=set()),
        num_scheduled_tokens={"q": 22}, preempted_req_ids=set()))
    loads = [(r, i.leases[0], list(i.block_ids_by_group[0])) for r, i in meta.load_intents.items()]
    assert loads == [("q", b"shard0-lease-001", [3, 4, 5])]
    saves = [("layer", list(i.block_ids_by_group[0]), list(i.block_hashes)) for i in meta.save_intents.values()]
    assert saves == [("layer", [6], [scripts.H(3)])]
