"""The engine as a sidecar process on a GPU: a worker process (this test) owns the KV cache, the
server (a child process, ``python -m pegaflow_b200.server``) maps it through CUDA IPC and moves the
bytes; everything between the two goes over gRPC with the reference's wire contract, the load's
completion through a shared-memory LoadState.  One layer travels as this library's IPC wrapper, one as
a pickle shaped like the reference's ``pegaflow.ipc_wrapper.CudaIPCWrapper`` (what an unmodified
reference connector sends)."""
import os
import pickle
import subprocess
import sys
import time
import types

import numpy as np
import pytest

from tests import scenarios as sc

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _reference_shaped_wrapper_bytes(torch, tensor):
    """A pickle that names `pegaflow.ipc_wrapper.CudaIPCWrapper` and carries the attributes the
    reference's class stores (python/pegaflow/ipc_wrapper.py:119-133)."""
    mod = types.ModuleType("pegaflow.ipc_wrapper")

    class CudaIPCWrapper:
        pass

    CudaIPCWrapper.__module__, CudaIPCWrapper.__qualname__ = "pegaflow.ipc_wrapper", "CudaIPCWrapper"
    mod.CudaIPCWrapper = CudaIPCWrapper
    saved = {k: sys.modules.get(k) for k in ("pegaflow", "pegaflow.ipc_wrapper")}
    sys.modules["pegaflow"] = sys.modules.get("pegaflow") or types.ModuleType("pegaflow")
    sys.modules["pegaflow.ipc_wrapper"] = mod
    try:
        w = CudaIPCWrapper()
        w.handle = tensor.untyped_storage()._share_cuda_()
        w.dtype, w.shape, w.stride, w.storage_offset = tensor.dtype, tensor.shape, tensor.stride(), 0
        w.device_uuid = str(torch.cuda.get_device_properties(tensor.device.index).uuid)
        return pickle.dumps(w)
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v


def test_worker_and_sidecar_in_two_processes():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("this test needs a CUDA device")
    import pegaflow_b200 as pf
    from pegaflow_b200.ipc import CudaIPCWrapper
    from pegaflow_b200.rpc_client import EngineRpcClient

    server = subprocess.Popen([sys.executable, "-m", "pegaflow_b200.server", "--addr", "127.0.0.1:0", "--pool-size", "64mb",
                               "--http-addr", "127.0.0.1:0"],
                              cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    try:
        line = server.stdout.readline()
        assert "listening on port" in line, line + server.stderr.read()[-2000:]
        client = EngineRpcClient(f"http://127.0.0.1:{int(line.split()[-1])}", timeout=60)
        assert client.health() == (True, "")
        http_line = server.stdout.readline()
        assert "HTTP endpoints on port" in http_line, http_line
        http_base = f"http://127.0.0.1:{int(http_line.split()[-1])}"

        dev = torch.device("cuda", 0)
        nb, seg = 64, 16 * 2 * 128 * 2
        caches = [torch.empty((2, nb, seg), dtype=torch.uint8, device=dev) for _ in range(2)]
        for i, t in enumerate(caches):
            t.copy_(torch.from_numpy(sc.seeded_bytes(2 * nb * seg, 80 + i).reshape(2, nb, seg)))
        torch.cuda.synchronize()
        before = [t.cpu().numpy().copy() for t in caches]
        names = ["model.layers.0.attn", "model.layers.1.attn"]
        wrappers = [CudaIPCWrapper(caches[0]).to_bytes(), _reference_shaped_wrapper_bytes(torch, caches[1])]
        assert client.register_context_batch("w", "ns", 0, 0, 1, 1, 0, names, wrappers, [nb] * 2, [seg] * 2, [nb * seg] * 2,
                                             [2] * 2, "direct", False) == (True, "")
        client.start_session_watcher("w", "ns", 1, 1)
        hashes = sc.make_block_hashes(5, 3)
        save_ids, load_ids = [3, 9, 40, 2, 17], [60, 61, 62, 63, 50]
        assert client.save("w", 0, 0, 0, [(n, save_ids, hashes) for n in names]) == (True, "")
        q = client.query_prefetch("w", hashes + [b"never-saved"], "req")
        assert q.num_hit_blocks == 5 and len(q.lease) == 16
        state = pf.PyLoadState()
        assert client.load("w", 0, 0, state.shm_name(), [names], [(q.lease, [load_ids])]) == (True, "")
        deadline = time.time() + 30
        while not state.is_ready() and time.time() < deadline:
            time.sleep(0.005)
        assert state.get_state() == 1
        torch.cuda.synchronize()
        for t, b in zip(caches, before):          # the other process wrote into this process's memory
            want = b.copy()
            want[:, load_ids] = b[:, save_ids]
            assert np.array_equal(t.cpu().numpy(), want)
        with pytest.raises(ValueError, match="out of range"):
            client.save("w", 0, 0, 0, [(names[0], [nb], [b"x"])])
        # the HTTP side of the same process: the real engine's counters under the reference's metric names
        import json
        import urllib.request

        assert urllib.request.urlopen(http_base + "/health", timeout=10).read() == b"ok"
        assert json.loads(urllib.request.urlopen(http_base + "/instances", timeout=10).read()) == {"instances": ["w"]}
        metrics = dict(line.split() for line in urllib.request.urlopen(http_base + "/metrics", timeout=10).read().decode()
                       .splitlines() if not line.startswith("#"))
        moved = 2 * 2 * 5 * seg                      # two layers, K and V, five blocks
        assert int(metrics["pegaflow_save_bytes_total"]) >= moved and int(metrics["pegaflow_load_bytes_total"]) == moved
        assert int(metrics["pegaflow_load_failures_total"]) == 0 and int(metrics["pegaflow_pool_capacity_bytes"]) >= 60 << 20
        assert 0 < int(metrics["pegaflow_pool_used_bytes"]) <= int(metrics["pegaflow_pool_capacity_bytes"])
        cleanup = urllib.request.Request(http_base + "/cache/memory/cleanup", data=b"", method="POST")
        stats = json.loads(urllib.request.urlopen(cleanup, timeout=10).read())
        assert stats["evicted_blocks"] == 5 and stats["still_referenced_blocks"] == 0 and stats["reclaimed_bytes"] > 0
        assert client.query_prefetch("w", hashes, "after-cleanup").num_hit_blocks == 0
        # this process "dies": the stream closes and the server lets the instance and its mappings go
        client.close()
        probe = EngineRpcClient(f"http://127.0.0.1:{int(line.split()[-1])}", timeout=60)
        deadline = time.time() + 10
        gone = False
        while not gone and time.time() < deadline:
            try:
                probe.query_prefetch("w", hashes, "after")
                time.sleep(0.1)
            except pf.PegaFlowError as e:
                gone = "instance w not found" in str(e)
        assert gone, "the session's end did not unregister the instance"
        assert probe.shutdown() == (True, "")
        probe.close()
        assert server.wait(timeout=30) == 0
    finally:
        if server.poll() is None:
            server.kill()
