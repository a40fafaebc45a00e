"""Case lists for the connector configuration helpers, shared by the fixture generator (which runs
them on the reference's module) and the test (which runs them on this package's module): the same
seeded inputs, the same way of recording answers and errors."""
import os
from types import SimpleNamespace


def _record(fn):
    try:
        return {"ok": fn()}
    except ValueError as e:
        return {"error": str(e)}


def fake_vllm_config(spec):
    model = SimpleNamespace(
        model=spec["model"], dtype=spec["dtype"],
        get_total_num_kv_heads=lambda: spec["kv_heads"], get_head_size=lambda: spec["head_size"],
        get_total_num_hidden_layers=lambda: spec["layers"],
        hf_text_config=SimpleNamespace(**({"kv_lora_rank": spec["kv_lora_rank"]} if "kv_lora_rank" in spec else {})))
    return SimpleNamespace(
        model_config=model, cache_config=SimpleNamespace(cache_dtype=spec["cache_dtype"]),
        parallel_config=SimpleNamespace(pipeline_parallel_size=spec["pp"], data_parallel_size=spec["dp"],
                                        data_parallel_rank_local=spec["dp_rank_local"]),
        scheduler_config=SimpleNamespace(disable_hybrid_kv_cache_manager=spec["disable_hma"]),
        additional_config=spec["additional"], instance_id=spec["instance_id"],
        kv_transfer_config=SimpleNamespace(engine_id=spec["engine_id"]))


def config_specs(rng, n=40):
    specs = []
    for i in range(n):
        spec = dict(
            model=rng.choice(["meta-llama/Llama-3.1-8B", "Qwen/Qwen3-0.6B", "deepseek-ai/DeepSeek-V3", "/models/local"]),
            dtype=rng.choice(["torch.bfloat16", "torch.float16", "auto"]), kv_heads=rng.choice([1, 2, 8, 32]),
            head_size=rng.choice([64, 128, 576]), layers=rng.choice([28, 32, 61, 80]),
            cache_dtype=rng.choice(["auto", "fp8", "fp8_e4m3"]), pp=rng.choice([1, 2, 4]), dp=rng.choice([1, 1, 2, 4]),
            dp_rank_local=rng.choice([None, 0, 1, 3]), disable_hma=rng.choice([True, False]),
            additional=rng.choice([None, {}, {"mla_layer_split_kv_cache": True}, {"mla_layer_split_kv_cache": 0}]),
            instance_id=rng.choice(["", "vllm-abc", "i-42"]), engine_id=rng.choice([None, "", "engine-7"]),
            tp=rng.choice([1, 2, 8]), dcp=rng.choice([1, 2]), pcp=rng.choice([1, 2]), cross_layer=rng.choice([True, False]),
            env_instance=rng.choice(["", "from-env"]), dp_suffix=rng.choice([True, True, False]))
        if rng.random() < 0.3:
            spec["kv_lora_rank"] = rng.choice([None, 512])
        specs.append(spec)
    return specs


TOPOLOGIES = [
    ("http://a:1", None, 8, 8), ("http://a:1", ["http://a:1", "http://b:1"], 8, 16),
    ("d", ("x", "y", "z", "w"), 8, 8), ("d", ["x", "y"], 3, 4), ("d", ["x", "y"], 4, 3), ("d", ["x", "x"], 4, 4),
    ("d", ["x", ""], 4, 4), ("d", [], 4, 4), ("d", "x,y", 4, 4), ("d", ["x", 5], 4, 4), ("d", ["x"], 0, 1),
    ("d", ["x"], 1, 0), ("d", ["p", "q"], 2, 2),
]


def cache_group_configs():
    """(name, kv_cache_config) pairs built from vLLM's own spec classes."""
    import torch
    from vllm.v1.kv_cache_interface import (ChunkedLocalAttentionSpec, FullAttentionSpec, KVCacheGroupSpec, MambaSpec,
                                            MLAAttentionSpec, SlidingWindowSpec, UniformTypeKVCacheSpecs)

    def full(bs=16):
        return FullAttentionSpec(block_size=bs, num_kv_heads=8, head_size=128, dtype=torch.bfloat16)

    def mla(bs=64):
        return MLAAttentionSpec(block_size=bs, num_kv_heads=1, head_size=576, dtype=torch.bfloat16)

    def mamba(bs=16, mode="align"):
        return MambaSpec(block_size=bs, shapes=((4, 8),), dtypes=(torch.float32,), mamba_cache_mode=mode)

    def sliding(bs=16):
        return SlidingWindowSpec(block_size=bs, num_kv_heads=8, head_size=128, dtype=torch.bfloat16, sliding_window=128)

    def chunked(bs=16):
        return ChunkedLocalAttentionSpec(block_size=bs, num_kv_heads=8, head_size=128, dtype=torch.bfloat16,
                                         attention_chunk_size=256)

    def uniform(specs, bs=64):
        return UniformTypeKVCacheSpecs(block_size=bs, kv_cache_specs=specs)

    def cfg(*groups):
        return SimpleNamespace(kv_cache_groups=[KVCacheGroupSpec(layer_names=list(n), kv_cache_spec=s) for n, s in groups])

    return [
        ("none", None), ("empty", SimpleNamespace(kv_cache_groups=[])),
        ("full", cfg((["l0", "l1"], full()))), ("mla", cfg((["l0"], mla()))),
        ("sliding_alone", cfg((["l0"], sliding()))), ("chunked_alone", cfg((["l0"], chunked()))),
        ("mamba_alone", cfg((["m0"], mamba()))),
        ("uniform_mla", cfg((["l0", "l1"], uniform({"l0": mla(), "l1": mla()})))),
        ("uniform_mixed", cfg((["l0", "l1"], uniform({"l0": mla(), "l1": full(64)})))),
        ("uniform_empty", cfg((["l0"], uniform({})))),
        ("full_mamba", cfg((["a0", "a1"], full()), (["m0", "m1"], mamba()))),
        ("mamba_full_mamba", cfg((["m0"], mamba()), (["a0"], full()), (["m1", "m2"], mamba()))),
        ("mla_mamba", cfg((["a0"], mla(16)), (["m0"], mamba()))),
        ("full_full", cfg((["a0"], full()), (["a1"], full()))),
        ("mamba_mamba", cfg((["m0"], mamba()), (["m1"], mamba()))),
        ("full_sliding", cfg((["a0"], full()), (["s0"], sliding()))),
        ("full_mamba_none", cfg((["a0"], full()), (["m0"], mamba(mode="none")))),
        ("full_mamba_block_sizes", cfg((["a0"], full(16)), (["m0"], mamba(32)))),
        ("duplicate_layer", cfg((["a0", "x"], full()), (["x"], mamba()))),
        ("full_two_mamba_full", cfg((["a0"], full()), (["m0"], mamba()), (["m1"], mamba()), (["a1"], full()))),
    ]


def _record_runtime(fn):
    try:
        return {"ok": fn()}
    except RuntimeError as e:
        return {"error": str(e)}


def run_cache_groups(mod):
    out = []
    for name, config in cache_group_configs():
        def build():
            lay = mod.CacheGroupLayout.from_config(config)
            return {"layer_names": [list(n) for n in lay.layer_names], "hash_group_index": lay.hash_group_index,
                    "has_recurrent_state": lay.has_recurrent_state,
                    "recurrent_group_indices": sorted(lay.recurrent_group_indices),
                    "recurrent_layer_names": sorted(lay.recurrent_layer_names),
                    "storage_group_ids": list(lay.storage_group_ids), "group_count": lay.group_count,
                    "storage_group_of": [lay.storage_group_of(i) for i in range(lay.group_count)],
                    "layer_to_group": _record_runtime(lay.layer_to_group)}
        out.append({"in": name, "out": _record_runtime(build)})
    return out


def run_all(mod, rng):
    out = {"mode": [], "topology": [], "config": [], "hybrid": []}
    for value in ["read_write", " Save_Only ", "READ_WRITE", "write", "", None, 3, "save-only"]:
        out["mode"].append({"in": value, "out": _record(lambda: mod.PegaConnectorMode.from_config(value).value)})
    out["backend"] = []
    for is_mla in (True, False):
        for override in (None, "direct", "kernel", " Kernel ", "DIRECT", "bogus", "", "kernel2"):
            out["backend"].append({"in": [is_mla, override],
                                   "out": _record(lambda: mod.resolve_transfer_backend(is_mla, override))})
    for default, configured, tp, world in TOPOLOGIES:
        def build():
            t = mod.TpShardTopology.from_config(default, configured, tp, world)
            probes = {}
            for rank in (-1, 0, 1, tp - 1, tp):
                probes[str(rank)] = _record(lambda: [t.shard_index(rank), t.local_tp_rank(rank)])
            names = {str(s): _record(lambda: t.namespace("base", s)) for s in (-1, 0, 1, t.shard_count - 1, t.shard_count)}
            return {"endpoints": list(t.endpoints), "shard_count": t.shard_count, "local_tp_size": t.local_tp_size,
                    "local_world_size": t.local_world_size, "ranks": probes, "namespaces": names}
        out["topology"].append({"in": [default, list(configured) if isinstance(configured, tuple) else configured, tp, world],
                                "out": _record(build)})
    for spec in config_specs(rng):
        cfg = fake_vllm_config(spec)
        saved = os.environ.get("PEGAFLOW_INSTANCE_ID")
        os.environ["PEGAFLOW_INSTANCE_ID"] = spec["env_instance"]
        try:
            instance = mod.resolve_instance_id(cfg, spec["dp_suffix"])
        finally:
            if saved is None:
                os.environ.pop("PEGAFLOW_INSTANCE_ID", None)
            else:
                os.environ["PEGAFLOW_INSTANCE_ID"] = saved
        generated = not (spec["engine_id"] or spec["instance_id"] or spec["env_instance"])
        if generated:   # a fresh uuid: only its shape can be compared
            head, _, tail = instance.partition("_dp")
            instance = ["uuid", len(head), tail]
        out["config"].append({"in": spec, "instance_id": instance,
                              "namespace": mod.derive_namespace(cfg, spec["tp"], spec["dcp"], spec["pcp"], spec["cross_layer"]),
                              "namespace_defaults": mod.derive_namespace(cfg, spec["tp"]),
                              "is_mla": mod.detect_mla(cfg)})
    for _ in range(60):
        attention = rng.choice([0, 1, 3, 8, 16, 20, -1])
        groups = rng.choice([0, 1, 1, 2, 3])
        shards = rng.choice([1, 2])
        hits = [[sorted(rng.sample(range(20), rng.choice([0, 4, 10, 16, 18, 19]))) for _ in range(shards)] for _ in range(groups)]
        blocks, checkpoint, usable = mod.reconcile_hybrid_hit(attention, tuple(tuple(tuple(s) for s in g) for g in hits))
        out["hybrid"].append({"in": [attention, hits], "out": [blocks, checkpoint, sorted(usable)]})
    return out
