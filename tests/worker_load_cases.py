"""Load intents of hybrid (attention + recurrent-state) models, shared by the fixture generator (which
hands them to the reference's WorkerConnector.start_load_kv) and the test (which hands them to this
package's worker mirror): what ends up in the engine's load request, or which error is raised."""

# cache groups of the model: (kind, layer names); the attention group carries the block hashes
LAYOUTS = {
    "attn_mamba": [("full", ["attn.0", "attn.1"]), ("mamba", ["mamba.0"])],
    "mamba_attn_mamba": [("mamba", ["m.0"]), ("full", ["a.0", "a.1"]), ("mamba", ["m.1", "m.2"])],
}

# name -> (layout, shard index, shard count, registered layers in order, {req: intent}, expected error or None)
# intent = (block ids by group, leases per shard, tokens, hold or None)
# hold   = (leases[g][shard], hit positions[g][shard], checkpoint)
CASES = {
    "one_request_with_checkpoint": (
        "attn_mamba", 0, 1, ["attn.0", "mamba.0", "attn.1"],
        {"r": ([[5, 6, 7, 8], [None, None, None, 43]], ["prefix-0"], 64, ([["mem-0"]], [[[1, 3]]], 3))}),
    "checkpoint_in_the_middle_of_the_lease": (
        "attn_mamba", 0, 1, ["attn.0", "attn.1", "mamba.0"],
        {"r": ([[5, 6], [None, 41]], ["prefix-0"], 32, ([["mem-0"]], [[[0, 1, 3]]], 1))}),
    "two_requests_one_without_hold": (
        "attn_mamba", 0, 1, ["attn.0", "attn.1", "mamba.0"],
        {"a": ([[1, 2], [None, 12]], ["pa"], 32, ([["ma"]], [[[1]]], 1)),
         "b": ([[3], [13]], ["pb"], 16, None)}),
    "second_shard_of_two_and_two_recurrent_groups": (
        "mamba_attn_mamba", 1, 2, ["m.0", "a.0", "a.1", "m.1", "m.2"],
        {"t": ([[None, None, 13], [1, 2, 3], [None, None, 23]], ["p-s0", "p-s1"], 48,
               ([["g0-s0", "g0-s1"], ["g1-s0", "g1-s1"]], [[[0, 2, 4], [2, 4]], [[2, 3, 4], [1, 2]]], 2))}),
    "only_some_layers_registered": (
        "mamba_attn_mamba", 0, 1, ["a.1", "m.2"],
        {"t": ([[None, 12], [1, 2], [None, 22]], ["p"], 32, ([["g0"], ["g1"]], [[[1]], [[0, 1]]], 1))}),
    "lease_count_mismatch": (
        "attn_mamba", 0, 2, ["attn.0", "mamba.0"],
        {"r": ([[5], [40]], ["only-one"], 16, ([["m"]], [[[0]]], 0))}),
    "checkpoint_not_under_the_lease": (
        "attn_mamba", 0, 1, ["attn.0", "mamba.0"],
        {"r": ([[5, 6], [None, 41]], ["p"], 32, ([["m"]], [[[0]]], 1))}),
    "no_recurrent_destination": (
        "attn_mamba", 0, 1, ["attn.0", "mamba.0"],
        {"r": ([[5, 6], [None, None]], ["p"], 32, ([["m"]], [[[1]]], 1))}),
    "nothing_to_load": (
        "attn_mamba", 0, 1, ["attn.0", "mamba.0"],
        {"r": ([[None], [None]], ["p"], 16, None)}),
}


def kv_cache_config(layout_name):
    """The layout as a vLLM KV-cache config built from vLLM's own spec classes."""
    from types import SimpleNamespace

    import torch
    from vllm.v1.kv_cache_interface import FullAttentionSpec, KVCacheGroupSpec, MambaSpec

    groups = []
    for kind, names in LAYOUTS[layout_name]:
        spec = (FullAttentionSpec(block_size=16, num_kv_heads=8, head_size=128, dtype=torch.bfloat16) if kind == "full"
                else MambaSpec(block_size=16, shapes=((4, 8),), dtypes=(torch.float32,), mamba_cache_mode="align"))
        groups.append(KVCacheGroupSpec(layer_names=list(names), kv_cache_spec=spec))
    return SimpleNamespace(kv_cache_groups=groups)


class RecordingClient:
    def __init__(self):
        self.calls = []

    def load(self, instance_id, tp_rank, device_id, shm_name, layer_groups, loads):
        self.calls.append({"layer_groups": [list(g) for g in layer_groups],
                           "loads": [[bytes(lease).decode(), [list(g) for g in ids]] for lease, ids in loads]})
        return True, ""

    def release(self, lease):
        self.calls.append({"release": bytes(lease).decode()})


def build_intents(spec, load_intent_cls, hold_cls):
    out = {}
    for req_id, (ids, leases, tokens, hold) in spec.items():
        h = None
        if hold is not None:
            h = hold_cls(leases=tuple(tuple(x.encode() for x in g) for g in hold[0]),
                         hit_positions=tuple(tuple(tuple(p) for p in g) for g in hold[1]), checkpoint=hold[2])
        out[req_id] = load_intent_cls(block_ids_by_group=tuple(tuple(g) for g in ids),
                                      leases=tuple(x.encode() for x in leases), num_tokens=tokens, recurrent_hold=h)
    return out


def run_all(start_load):
    """`start_load(layout name, shard index, shard count, registered layers, intent spec, client)` drives one
    implementation; the record is what reached the engine client, or the error raised."""
    results = {}
    for name, (layout, shard, shards, layers, intents) in CASES.items():
        client = RecordingClient()
        try:
            start_load(layout, shard, shards, layers, intents, client)
            outcome = {"calls": client.calls}
        except RuntimeError as e:
            outcome = {"error": str(e), "calls": client.calls}
        results[name] = outcome
    return results
