"""The connector configuration helpers (pegaflow_b200/config.py) give the reference's answers:
the committed fixture holds what the reference's own python/pegaflow/connector/common.py returned
for the shared case lists (tests/golden/gen_connector_config.py), error messages included."""
import json
import os
import random

from pegaflow_b200 import config as mine
from tests import connector_config_cases as cases

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _golden():
    return json.load(open(os.path.join(ROOT, "tests", "golden", "connector_config.json")))


def _as_json(obj):
    return json.loads(json.dumps(obj, sort_keys=True))


def test_every_case_list_matches_the_reference():
    golden = _golden()
    got = cases.run_all(mine, random.Random(20260101))
    try:
        got["cache_groups"] = cases.run_cache_groups(mine)     # built from vLLM's own spec classes
    except ImportError:
        golden.pop("cache_groups")
    got = _as_json(got)
    assert set(got) == set(golden)
    for section in golden:
        assert len(got[section]) == len(golden[section]) and len(golden[section]) >= 8
        for i, (a, b) in enumerate(zip(got[section], golden[section])):
            assert a == b, f"{section}[{i}]: {a} != {b}"


def test_fixture_covers_the_interesting_outcomes():
    golden = _golden()
    assert sum(1 for h in golden["hybrid"] if h["out"][0] > 0) >= 10
    assert sum(1 for h in golden["hybrid"] if h["out"][0] == 0) >= 10
    assert any("error" in t["out"] for t in golden["topology"]) and any("ok" in t["out"] for t in golden["topology"])
    assert len({c["namespace"] for c in golden["config"]}) >= 35, "namespaces should separate different layouts"
    assert any(isinstance(c["instance_id"], list) for c in golden["config"]), "a generated id should be among the cases"
    assert any(c["is_mla"] for c in golden["config"])


def test_namespace_changes_with_every_layout_factor():
    rng = random.Random(7)
    spec = cases.config_specs(rng, 1)[0]
    base = mine.derive_namespace(cases.fake_vllm_config(spec), 2)
    for key, other in [("model", "x/y"), ("dtype", "torch.float32"), ("kv_heads", 5), ("head_size", 96), ("layers", 7),
                       ("cache_dtype", "fp8_e5m2"), ("pp", 8), ("disable_hma", not spec["disable_hma"]),
                       ("additional", {"mla_layer_split_kv_cache": not bool((spec["additional"] or {}).get(
                           "mla_layer_split_kv_cache", False))})]:
        changed = dict(spec, **{key: other})
        assert mine.derive_namespace(cases.fake_vllm_config(changed), 2) != base, key
    cfg = cases.fake_vllm_config(spec)
    assert mine.derive_namespace(cfg, 4) != base
    assert mine.derive_namespace(cfg, 2, dcp_world_size=2) != base
    assert mine.derive_namespace(cfg, 2, pcp_world_size=2) != base
    assert mine.derive_namespace(cfg, 2, cross_layer_blocks=True) != base
