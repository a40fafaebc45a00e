"""One vLLM process with this library as its KV connector (run by tests/test_gpu_vllm.py in a
subprocess; prints one JSON line).

A small randomly initialised Llama runs three times over the same prompts: cold (computes the
prompt, the connector saves its KV blocks), warm from vLLM's own GPU prefix cache, and — after that
cache has been reset — warm from the host pool through the connector.  The two warm runs take the
same compute path for the remaining token, so their sampled tokens and log-probabilities must be
identical if the loaded KV bytes are the saved ones and no layer was read before it had landed.
"""
import json
import os
import sys
import tempfile

os.environ.setdefault("VLLM_ENABLE_V1_MULTIPROCESSING", "0")
os.environ.setdefault("VLLM_LOGGING_LEVEL", "WARNING")
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


class Sidecar:
    """``python -m pegaflow_b200.server`` as a child process; its counters are read over HTTP."""

    def __init__(self):
        import subprocess

        root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
        self.proc = subprocess.Popen([sys.executable, "-m", "pegaflow_b200.server", "--addr", "127.0.0.1:0", "--http-addr",
                                      "127.0.0.1:0", "--pool-size", "1gb"], cwd=root, stdout=subprocess.PIPE, text=True)
        self.port = int(self.proc.stdout.readline().split()[-1])
        self.http = f"http://127.0.0.1:{int(self.proc.stdout.readline().split()[-1])}"

    def metrics(self):
        import urllib.request

        text = urllib.request.urlopen(self.http + "/metrics", timeout=30).read().decode()
        raw = dict(line.split() for line in text.splitlines() if not line.startswith("#"))
        return {"save_bytes": int(raw["pegaflow_save_bytes_total"]), "load_bytes": int(raw["pegaflow_load_bytes_total"]),
                "load_failures": int(raw["pegaflow_load_failures_total"]), "cache_blocks": None}

    def stop(self):
        self.proc.kill()
        try:
            self.proc.wait(10)
        except Exception:
            pass


def main():
    sidecar = Sidecar() if "--sidecar" in sys.argv else None
    layerwise = "--after-forward" not in sys.argv and sidecar is None
    import numpy as np
    from transformers import LlamaConfig
    from vllm import LLM, SamplingParams
    from vllm.config import KVTransferConfig

    from pegaflow_b200 import vllm_connector

    model_dir = tempfile.mkdtemp(prefix="tiny-llama-")
    LlamaConfig(vocab_size=2048, hidden_size=512, intermediate_size=1024, num_hidden_layers=4, num_attention_heads=8,
                num_key_value_heads=2, head_dim=64, max_position_embeddings=4096, torch_dtype="bfloat16",
                architectures=["LlamaForCausalLM"]).save_pretrained(model_dir)
    try:
        llm = _start(LLM, KVTransferConfig, model_dir, layerwise, sidecar)
    except Exception:
        import traceback

        tb = traceback.format_exc()
        # an engine that cannot start for reasons outside this library (no free port, no shared
        # memory, an incompatible vLLM build) is not a verdict on the connector
        print(json.dumps({"engine_start_failed": True, "ours": "pegaflow_b200" in tb, "traceback": tb[-2000:]}))
        sys.stdout.flush()
        if sidecar:
            sidecar.stop()
        import multiprocessing

        for child in multiprocessing.active_children():
            child.terminate()
        os._exit(0)
    _scenario(llm, SamplingParams, vllm_connector, layerwise, np, sidecar)


def _tp_size():
    return int(sys.argv[sys.argv.index("--tp") + 1]) if "--tp" in sys.argv else 1


def _start(LLM, KVTransferConfig, model_dir, layerwise, sidecar=None):
    extra = {"pegaflow.pool_bytes": 1 << 30, "pegaflow.layerwise": layerwise}
    if sidecar:
        extra = {"pegaflow.host": "http://127.0.0.1", "pegaflow.port": sidecar.port}
    parallel = {}
    if _tp_size() > 1:
        # worker processes, one per GPU; vLLM's own all-reduce goes through NCCL only
        parallel = dict(tensor_parallel_size=_tp_size(), distributed_executor_backend="mp", disable_custom_all_reduce=True)
    return LLM(**parallel, model=model_dir, load_format="dummy", skip_tokenizer_init=True,
               enforce_eager="--cuda-graphs" not in sys.argv, max_model_len=2048,
              gpu_memory_utilization=0.10, dtype="bfloat16", seed=0, enable_prefix_caching=True, block_size=16,
              kv_transfer_config=KVTransferConfig(
                  kv_connector="PegaKVConnector", kv_connector_module_path="pegaflow_b200.vllm_connector", kv_role="kv_both",
                  kv_connector_extra_config=extra))


def _scenario(llm, SamplingParams, vllm_connector, layerwise, np, sidecar=None):
    rng = np.random.default_rng(3)
    prompts = [{"prompt_token_ids": rng.integers(1, 2000, size=n).tolist()} for n in (200, 333, 64, 1000)]
    params = SamplingParams(temperature=0.0, max_tokens=6, detokenize=False, logprobs=1)

    def run():
        outs = llm.generate(prompts, params, use_tqdm=False)
        return [[(int(t), float(next(iter(lp.values())).logprob)) for t, lp in zip(o.outputs[0].token_ids, o.outputs[0].logprobs)]
                for o in outs]

    engine = sidecar or next(iter(vllm_connector._ENGINES.values()))
    cold = run()
    after_cold = engine.metrics()
    gpu_cache = run()
    after_gpu_cache = engine.metrics()
    # A request whose last save happened in its final steps keeps its blocks until the worker has
    # reported the save as sent, which takes one more engine step; then nothing is in use any more.
    llm.generate([{"prompt_token_ids": [5, 6, 7]}], SamplingParams(temperature=0.0, max_tokens=1, detokenize=False),
                 use_tqdm=False)
    reset_ok = llm.reset_prefix_cache()
    host_pool = run()
    after_host = engine.metrics()
    print(json.dumps({
        "layerwise": layerwise, "sidecar": sidecar is not None, "tp": _tp_size(), "cuda_graphs": "--cuda-graphs" in sys.argv,
        "prefix_cache_reset": bool(reset_ok),
        "warm_runs_identical": gpu_cache == host_pool, "cold_equals_warm_tokens": [[t for t, _ in a] for a in cold] ==
        [[t for t, _ in a] for a in host_pool],
        "saved_bytes_cold": after_cold["save_bytes"], "loaded_bytes_gpu_cache_run": after_gpu_cache["load_bytes"],
        "loaded_bytes_host_pool_run": after_host["load_bytes"] - after_gpu_cache["load_bytes"],
        "load_failures": after_host["load_failures"], "cache_blocks": after_host["cache_blocks"],
        "tokens": [[t for t, _ in a] for a in host_pool]}))
    sys.stdout.flush()
    vllm_connector.close_shared_engines()
    if _tp_size() > 1:
        _stop_workers(llm)
    if sidecar:
        sidecar.stop()
    os._exit(0)      # vLLM's own teardown is not what this scenario tests


def _stop_workers(llm):
    """Worker processes must not outlive this one: ask the executor to stop them, then make sure."""
    import multiprocessing

    try:
        llm.llm_engine.engine_core.shutdown()
    except Exception:
        pass
    for child in multiprocessing.active_children():
        child.terminate()
    for child in multiprocessing.active_children():
        child.join(10)


if __name__ == "__main__":
    main()
