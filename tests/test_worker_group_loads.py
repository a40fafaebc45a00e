"""Loads of models with several cache groups: the worker mirror sends the engine exactly the load
requests the reference's worker sends (tests/golden/worker_loads.json, recorded by
tests/golden/gen_worker_loads.py), and refuses what it refuses with the same words.  Host logic
only: the engine client is a recorder."""
import json
import os

import pytest

from tests import worker_load_cases as cases

HERE = os.path.dirname(os.path.abspath(__file__))


def _start_load(layout, shard, shards, layers, intents, client):
    pytest.importorskip("vllm")
    from pegaflow_b200.config import CacheGroupLayout
    from pegaflow_b200.connector import PegaWorkerConnector
    from pegaflow_b200.scheduler import LoadIntent, PegaConnectorMetadata, RecurrentLoadHold

    worker = PegaWorkerConnector(client, None, instance_id="inst", namespace="ns", device_id=0, block_size=16,
                                 tp_rank=0, tp_size=1, cache_groups=CacheGroupLayout.from_config(cases.kv_cache_config(layout)),
                                 tp_shard_count=shards)
    worker.registered_layers = list(layers)
    meta = PegaConnectorMetadata(load_intents=cases.build_intents(intents, LoadIntent, RecurrentLoadHold))
    worker.start_load_kv_from_metadata(meta, shard_index=shard)
    return worker


def test_group_loads_match_the_reference_worker():
    golden = json.load(open(os.path.join(HERE, "golden", "worker_loads.json")))
    got = json.loads(json.dumps(cases.run_all(_start_load)))
    assert sorted(got) == sorted(golden) and len(golden) >= 9
    for name in golden:
        assert got[name] == golden[name], f"{name}:\n{got[name]}\n{golden[name]}"
    assert sum(1 for v in golden.values() if "error" in v) == 3
    two = golden["second_shard_of_two_and_two_recurrent_groups"]["calls"][0]
    assert [lease for lease, _ in two["loads"]] == ["p-s1", "g0-s1", "g1-s1"], "the second shard's leases"


def test_a_group_load_that_cannot_be_submitted_raises_after_giving_the_leases_back():
    """worker.py:650-684: with several cache groups vLLM cannot recompute a failed load."""
    class Refusing(cases.RecordingClient):
        def load(self, *a):
            super().load(*a)
            return False, "engine restarting"

    client = Refusing()
    with pytest.raises(RuntimeError, match="HMA load failed.*engine restarting"):
        _start_load(*cases.CASES["one_request_with_checkpoint"], client)
    assert [c["release"] for c in client.calls if "release" in c] == ["prefix-0", "mem-0"]


def test_saves_take_each_layer_s_own_group_ids():
    """worker.py:850-866: a layer saves the ids of its cache group; the null block (id 0) that pads a
    recurrent group's positions before the state block is never saved."""
    pytest.importorskip("vllm")
    from pegaflow_b200.config import CacheGroupLayout
    from pegaflow_b200.connector import PegaWorkerConnector
    from pegaflow_b200.scheduler import PegaConnectorMetadata, SaveIntent

    class Saver(cases.RecordingClient):
        def save(self, instance_id, tp_rank, pp_rank, device_id, saves):
            self.calls.append({"save": [(n, list(i), [bytes(h).decode() for h in hs]) for n, i, hs in saves]})
            return True, ""

        def flush_saves(self):
            return True, ""

    client = Saver()
    worker = PegaWorkerConnector(client, None, instance_id="inst", namespace="ns", device_id=0, block_size=16,
                                 cache_groups=CacheGroupLayout.from_config(cases.kv_cache_config("attn_mamba")))
    worker.registered_layers = ["attn.0", "mamba.0", "attn.1"]
    intent = SaveIntent(((13, 14, 15), (0, 0, 36)), (b"h3", b"h4", b"h5"))
    done = worker.wait_for_save_from_metadata(PegaConnectorMetadata(ready_save_intents={"r": intent}))
    assert done == {"r"}
    (call,) = [c["save"] for c in client.calls if "save" in c]
    assert call == [("attn.0", [13, 14, 15], ["h3", "h4", "h5"]), ("mamba.0", [36], ["h5"]),
                    ("attn.1", [13, 14, 15], ["h3", "h4", "h5"])]
    with pytest.raises(RuntimeError, match="missing cache group 1"):
        worker.wait_for_save_from_metadata(PegaConnectorMetadata(save_intents={"r": SaveIntent(((1,),), (b"h",))}))
    with pytest.raises(RuntimeError, match="count mismatch"):
        worker.wait_for_save_from_metadata(PegaConnectorMetadata(save_intents={"r": SaveIntent(((1,), (2, 3)), (b"h",))}))


@pytest.mark.parametrize("how", ["error", "timeout"])
def test_a_group_load_that_fails_later_ends_the_step_like_the_reference(how):
    """worker.py:467-470, 499-503, 534-539: when the load state of a multi-group load reports an error,
    or the load outlives the timeout, the service is marked unavailable and get_finished raises; the
    blocks are not reported as invalid (vLLM could not recompute them for several groups)."""
    client = cases.RecordingClient()
    worker = _start_load(*cases.CASES["one_request_with_checkpoint"], client)
    (pending,) = worker._pending_loads
    assert worker.get_finished() == ([], [])            # still pending, within the timeout
    if how == "error":
        pending.state.set_error()
        match = r"HMA load failed.*async load failed for requests \[.*\]: state=-1"
    else:
        worker.LOAD_TIMEOUT_SECONDS = 0.0
        match = r"HMA load failed.*load timed out for requests \[.*\] after"
    with pytest.raises(RuntimeError, match=match):
        worker.get_finished()
    assert not worker.state_manager.is_available()
    assert worker.get_block_ids_with_load_errors() == set()
    assert worker._pending_loads == [] and worker.get_finished() == ([], [])   # reported once
    assert worker.load_history[-1][2] is False


def test_transfer_stats_have_the_reference_shape():
    """connector_metrics.py:115-260: keys, counters, list extension on aggregate, the logged summary, reset on read."""
    from pegaflow_b200.connector import TransferStats

    a, b = TransferStats(), TransferStats()
    assert a.is_empty() and a.reduce() == {"pending_save_requests": 0, "load_success_count": 0, "load_failure_count": 0,
                                          "save_success_count": 0, "save_failure_count": 0}
    a.record_load(0.010, 64, True)
    a.record_load(0.030, 16, False)
    b.record_save(0.002, 8, True)
    b.data["pending_save_requests"] = 3
    assert not a.is_empty() and not b.is_empty()
    merged = a.aggregate(b)
    assert merged is a and a.data["load_duration"] == [0.010, 0.030] and a.data["save_blocks"] == [8]
    assert a.reduce() == {"pending_save_requests": 3, "num_loads": 2, "avg_load_duration_ms": 20.0, "total_load_blocks": 80,
                          "avg_load_blocks": 40.0, "load_success_count": 1, "load_failure_count": 1, "num_saves": 1,
                          "avg_save_duration_ms": 2.0, "total_save_blocks": 8, "avg_save_blocks": 8.0,
                          "save_success_count": 1, "save_failure_count": 0}
    old = a.clone_and_reset()
    assert a.is_empty() and old.data["load_success_count"] == 1 and old.data["save_duration"] == [0.002]


def test_worker_records_its_loads_and_saves():
    """worker.py:525-528, 741-753, 925-926, 1039-1047: finished loads, loads that could not be submitted and batch
    saves each leave a record; a reading hands them out and starts afresh."""
    from pegaflow_b200.connector import PegaWorkerConnector

    class Client:
        def __init__(self):
            self.accept_loads = True

        def health(self):
            return True, ""

        def load(self, *a):
            return (True, "") if self.accept_loads else (False, "no")

        def release(self, lease):
            pass

        def save(self, instance_id, tp_rank, pp_rank, device_id, saves):
            return True, ""

        def flush_saves(self):
            return True, ""

    client = Client()
    w = PegaWorkerConnector(client, None, instance_id="i", namespace="n", device_id=0, block_size=16)
    w.registered_layers = ["layer_0", "layer_1"]
    assert w.get_stats() is None
    w.start_load_kv([("req-a", b"L" * 16, [4, None, 9])])
    w._pending_loads[0].state.set_completed()
    assert w.get_finished() == (["req-a"], [])
    client.accept_loads = False
    w.start_load_kv([("req-b", b"M" * 16, [1, 2, 3])])
    w.wait_for_save([("layer_0", [0, 5, 6], [b"z", b"a", b"b"]), ("layer_1", [5, 6], [b"a", b"b"])])
    got = w.get_stats()
    assert got.data["load_blocks"] == [2, 3] and got.data["load_success_count"] == 1 and got.data["load_failure_count"] == 1
    assert got.data["save_blocks"] == [4] and got.data["save_success_count"] == 1      # block 0 is vLLM's null block
    assert w.get_stats() is None
