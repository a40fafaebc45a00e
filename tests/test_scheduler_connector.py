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


def _make(clients, *, block_size, read_enabled, wait_for_full_prefix, group_count, recurrent_groups=0):
    from pegaflow_b200.config import CacheGroupLayout
    from pegaflow_b200.scheduler import SchedulerConnector

    assert group_count == 1
    layout = None
    if recurrent_groups:
        # one attention group followed by the recurrent-state groups, storage groups 1..n
        names = (("attn",),) + tuple((f"mamba{g}",) for g in range(1, recurrent_groups + 1))
        layout = CacheGroupLayout(names, 0, True, frozenset(range(1, recurrent_groups + 1)),
                                  frozenset(n for g in names[1:] for n in g), tuple(range(recurrent_groups + 1)))
    return SchedulerConnector(clients, instance_id="inst", block_size=block_size, read_enabled=read_enabled,
                              wait_for_full_prefix=wait_for_full_prefix, cache_groups=layout)


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


# ---- known answers from the reference's own unit tests (python/tests/test_tp_shards.py:196-306) -----------
def _mock_pair():
    from unittest.mock import MagicMock

    return MagicMock(), MagicMock()


def test_kat_common_prefix_and_exact_per_shard_leases():
    from unittest.mock import call

    from pegaflow_b200.connector import QueryReady
    from pegaflow_b200.scheduler import ShardQuery

    first, second = _mock_pair()
    first.query_prefetch.side_effect = [QueryReady(3, b"first-long"), QueryReady(2, b"first-exact")]
    second.query_prefetch.return_value = QueryReady(2, b"second-exact")
    hashes = [b"h0", b"h1", b"h2"]
    assert ShardQuery((first, second)).query("instance", hashes, "request", False) == (2, (b"first-exact", b"second-exact"))
    assert first.query_prefetch.call_args_list == [
        call("instance", hashes, req_id="request", wait_for_full_prefix=False),
        call("instance", hashes[:2], req_id="request:tp-common-2", wait_for_full_prefix=False)]
    first.release.assert_called_once_with(b"first-long")
    second.release.assert_not_called()


def test_kat_ready_shards_are_released_when_another_is_loading():
    from pegaflow_b200.connector import QueryLoading, QueryReady
    from pegaflow_b200.scheduler import ShardQuery

    first, second = _mock_pair()
    first.query_prefetch.return_value = QueryReady(2, b"first")
    second.query_prefetch.return_value = QueryLoading()
    assert ShardQuery((first, second)).query("instance", [b"h0", b"h1"], "request", False) is None
    first.release.assert_called_once_with(b"first")


def test_kat_drifted_prefetch_is_discarded_before_new_hashes_are_queried():
    from types import SimpleNamespace
    from unittest.mock import call

    from pegaflow_b200.connector import QueryLoading, QueryReady
    from pegaflow_b200.scheduler import SchedulerConnector

    first, second = _mock_pair()
    first.query_prefetch.side_effect = [QueryLoading(), QueryReady(4, b"first-old"), QueryLoading()]
    second.query_prefetch.return_value = QueryReady(4, b"second-old")
    sched = SchedulerConnector((first, second), instance_id="instance", block_size=16)
    request = SimpleNamespace(request_id="request", block_hashes=[b"h0", b"h1", b"h2", b"h3"], num_tokens=64)
    assert sched.get_num_new_matched_tokens(request, 0) == (None, False)
    assert sched.get_num_new_matched_tokens(request, 32) == (None, False)
    assert sched.get_num_new_matched_tokens(request, 32) == (None, False)
    old, new = request.block_hashes, request.block_hashes[2:]
    assert first.query_prefetch.call_args_list == [
        call("instance", old, req_id="request", wait_for_full_prefix=False),
        call("instance", old, req_id="request", wait_for_full_prefix=False),
        call("instance", new, req_id="request", wait_for_full_prefix=False)]
    first.release.assert_called_once_with(b"first-old")
    second.release.assert_called_once_with(b"second-old")


@pytest.mark.parametrize("hits,lease", [(3, b"too-many"), (1, b"")])
def test_kat_invalid_shard_answers_do_not_leak_leases(hits, lease):
    from pegaflow_b200.connector import QueryReady
    from pegaflow_b200.scheduler import ShardQuery

    first, second = _mock_pair()
    first.query_prefetch.return_value = QueryReady(2, b"first")
    second.query_prefetch.return_value = QueryReady(hits, lease)
    with pytest.raises(RuntimeError, match="TP shard 1"):
        ShardQuery((first, second)).query("instance", [b"h0", b"h1"], "request", False)
    first.release.assert_called_once_with(b"first")
    if lease:
        second.release.assert_called_once_with(lease)


# ---- which KV-cache group layouts are served (python/tests/test_cache_group_layout.py:72-135) ---------------
def _spec(name, **attrs):
    return type(name, (), {})() if not attrs else type(name, (), attrs)()


def _cfg(*specs):
    from types import SimpleNamespace

    return SimpleNamespace(kv_cache_groups=[SimpleNamespace(layer_names=("l",), kv_cache_spec=s) for s in specs])


def test_single_attention_or_mla_groups_are_accepted():
    from pegaflow_b200.scheduler import require_single_attention_group as check

    check(None)
    check(_cfg())
    check(_cfg(_spec("FullAttentionSpec")))
    check(_cfg(_spec("MLAAttentionSpec")))
    check(_cfg(_spec("UniformTypeKVCacheSpecs", kv_cache_specs={"a": _spec("MLAAttentionSpec"), "b": _spec("MLAAttentionSpec")})))


@pytest.mark.parametrize("specs", [
    (_spec("MambaSpec"),), (_spec("SlidingWindowSpec"),),
    (_spec("UniformTypeKVCacheSpecs", kv_cache_specs={}),),
    (_spec("UniformTypeKVCacheSpecs", kv_cache_specs={"a": _spec("MLAAttentionSpec"), "b": _spec("FullAttentionSpec")}),),
    (_spec("FullAttentionSpec"), _spec("MambaSpec")),
    (_spec("FullAttentionSpec"), _spec("FullAttentionSpec")),
])
def test_other_group_layouts_are_refused(specs):
    from pegaflow_b200.scheduler import require_single_attention_group as check

    with pytest.raises(RuntimeError, match="single"):
        check(_cfg(*specs))


# ---- ShardQuery against recorded answers of the reference's TpShardQueryClient -----------------------------
def test_shard_query_replays_the_reference_in_scripted_scenarios():
    """tests/golden/shard_query.json holds, for 150 scripted scenarios (70 prefix and membership queries, 80 hybrid lookups; shards that answer Ready with
    varying hit counts, Loading, raise, return malformed answers, or fail to release), what the
    reference's client returned or raised and every call it made to the shards, in order.  The
    mirror must do exactly the same: same result, same exception type and text, same queries,
    same releases."""
    import json
    import os

    from pegaflow_b200.connector import QueryLoading, QueryReady
    from pegaflow_b200.scheduler import ShardQuery
    from tests import shard_query_cases as cases

    class Adapter:
        def __init__(self, shards):
            self.client = ShardQuery(shards)

        def prefix(self, instance_id, hashes, req_id, wait):
            got = self.client.query(instance_id, hashes, req_id, wait)
            return None if got is None else [got[0], [lease.decode() for lease in got[1]]]

        def membership(self, instance_id, hashes, req_id, group_id):
            return [[list(p), lease.decode()]
                    for p, lease in self.client.query_group_membership(instance_id, hashes, req_id, group_id)]

    def hybrid_adapter(shards, group_ids):
        client = ShardQuery(shards)

        class H:
            def hybrid(self, instance_id, hashes, req_id, wait):
                got = client.query_hybrid(instance_id, hashes, req_id, wait, group_ids)
                if got is None:
                    return None
                return {"hit": got.num_hit_blocks, "leases": [x.decode() for x in got.leases],
                        "recurrent_leases": [[x.decode() for x in g] for g in got.recurrent_leases],
                        "recurrent_positions": [[list(p) for p in g] for g in got.recurrent_positions],
                        "checkpoint": got.checkpoint, "usable": list(got.usable_positions)}
        return H()

    here = os.path.dirname(os.path.abspath(__file__))
    golden = json.load(open(os.path.join(here, "golden", "shard_query.json")))
    got = cases.run_all(Adapter, QueryReady, QueryLoading) + cases.run_hybrid(hybrid_adapter, QueryReady, QueryLoading)
    got = json.loads(json.dumps(got))
    assert len(got) == len(golden) == 150
    kinds = set()
    for i, (a, b) in enumerate(zip(got, golden)):
        assert a["scripts"] == b["scripts"], f"scenario {i}: the scripts differ, regenerate the fixture"
        assert a["outcome"] == b["outcome"], f"scenario {i} ({a['kind']}): {a['outcome']} != {b['outcome']}"
        assert a["log"] == b["log"], f"scenario {i} ({a['kind']}): calls differ\n{a['log']}\n{b['log']}"
        kinds.add((b["kind"], "ok" if "ok" in b["outcome"] else b["outcome"]["error"][0]))
    assert {("prefix", "ok"), ("prefix", "RuntimeError"), ("prefix", "ConnectionError"), ("membership", "ok"),
            ("membership", "RuntimeError"), ("hybrid", "ok"), ("hybrid", "RuntimeError"),
            ("hybrid", "ConnectionError")} <= kinds
    hybrid_ok = [b["outcome"]["ok"] for b in golden if b["kind"] == "hybrid" and b["outcome"].get("ok")]
    assert sum(1 for h in hybrid_ok if h["hit"] > 0) >= 10, "the fixture should hold real hybrid hits"
    assert any(h["hit"] > 0 and h["leases"][0].endswith("-x") for h in hybrid_ok), "and re-leased shortened prefixes"
