"""This library as the KV connector of a real vLLM engine (the reference's
python/tests/test_vllm_e2e_correctness.py idea, with a randomly initialised model): prompts served
warm from the host pool must produce exactly what the same prompts produce warm from vLLM's own GPU
prefix cache."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("mode", ["layerwise", "after-forward", "sidecar"])
def test_vllm_serves_prompts_from_the_host_pool(mode):
    pytest.importorskip("vllm")
    if os.environ.get("PEGAFLOW_TEST_VLLM", "1") == "0":
        pytest.skip("PEGAFLOW_TEST_VLLM=0: not starting a vLLM engine (it takes about a minute per mode)")
    import torch

    if not torch.cuda.is_available():
        pytest.fail("this test needs a CUDA device")
    # "sidecar": the engine in a server process of its own, reached over gRPC and CUDA IPC like the reference's
    cmd = [sys.executable, os.path.join(HERE, "vllm_scenario.py")] + {"after-forward": ["--after-forward"],
                                                                       "sidecar": ["--sidecar"]}.get(mode, [])
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=900)
    lines = [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]
    assert proc.returncode == 0 and lines, proc.stderr[-3000:]
    out = json.loads(lines[-1])
    if out.get("engine_start_failed"):
        assert not out["ours"], out["traceback"]
        pytest.skip("the vLLM engine could not start here: " + out["traceback"].strip().splitlines()[-1])
    assert out["saved_bytes_cold"] > 0, "the cold run saved nothing"
    assert out["prefix_cache_reset"], "vLLM could not reset its prefix cache: some request still holds blocks"
    # the GPU-cache run only asks the pool for what vLLM's own cache left over (at most a block per prompt)
    assert out["loaded_bytes_host_pool_run"] > 10 * max(1, out["loaded_bytes_gpu_cache_run"]), \
        "the third run did not load the prompts from the host pool"
    assert out["load_failures"] == 0
    assert out["warm_runs_identical"], "tokens or log-probabilities differ between GPU-cache and host-pool warm runs"


def test_vllm_tensor_parallel_workers_through_the_sidecar():
    """Two tensor-parallel worker processes, one per GPU, against one server process: each registers its shard of
    the KV cache under its own rank, a block is a hit once both ranks have saved it, each rank loads its own slots
    (the reference's deployment, pegaflow-server/tests/mock_vllm_rpc_e2e.rs:318-360 with a real vLLM)."""
    pytest.importorskip("vllm")
    if os.environ.get("PEGAFLOW_TEST_VLLM", "1") == "0":
        pytest.skip("PEGAFLOW_TEST_VLLM=0: not starting a vLLM engine")
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    cmd = [sys.executable, os.path.join(HERE, "vllm_scenario.py"), "--sidecar", "--tp", "2"]
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=900)
    lines = [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]
    assert proc.returncode == 0 and lines, proc.stderr[-3000:]
    out = json.loads(lines[-1])
    if out.get("engine_start_failed"):
        assert not out["ours"], out["traceback"]
        pytest.skip("the vLLM engine could not start here: " + out["traceback"].strip().splitlines()[-1])
    assert out["tp"] == 2 and out["sidecar"]
    assert out["saved_bytes_cold"] > 0 and out["prefix_cache_reset"]
    assert out["loaded_bytes_host_pool_run"] > 10 * max(1, out["loaded_bytes_gpu_cache_run"])
    assert out["load_failures"] == 0
    assert out["warm_runs_identical"], "tokens or log-probabilities differ between GPU-cache and host-pool warm runs"
