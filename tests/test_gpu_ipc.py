"""Cross-process registration: a worker process owns the KV cache, the engine runs in another
process and reaches the same GPU memory through CUDA IPC (the reference's worker / sidecar split,
python/pegaflow/ipc_wrapper.py + pegaflow-server/src/registry.rs)."""
import json
import os
import pickle
import subprocess
import sys
import tempfile

import numpy as np
import pytest

from tests import scenarios as sc

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def test_engine_in_another_process_saves_and_loads_through_ipc():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("this test needs a CUDA device")
    from pegaflow_b200.ipc import CudaIPCWrapper

    dev = torch.device("cuda", 0)
    nb, seg, n_layers = 64, 16 * 2 * 128 * 2, 3
    # HND-ordered view of NHD storage for one layer: the wrapper carries the storage, not the view
    caches = [torch.empty((2, nb, 16, 2, 128), dtype=torch.bfloat16, device=dev) for _ in range(n_layers)]
    caches[1] = torch.empty((2, nb, 2, 16, 128), dtype=torch.bfloat16, device=dev).permute(0, 1, 3, 2, 4)
    for i, t in enumerate(caches):
        torch.empty(0, dtype=torch.uint8, device=dev).set_(t.untyped_storage()).random_(
            0, 256, generator=torch.Generator(device=dev).manual_seed(70 + i))
    torch.cuda.synchronize()

    def storage_bytes(t):
        return torch.empty(0, dtype=torch.uint8, device=dev).set_(t.untyped_storage()).cpu().numpy().copy()

    before = [storage_bytes(t) for t in caches]
    wrappers = [CudaIPCWrapper(t) for t in caches]
    assert pickle.loads(pickle.dumps(wrappers[0])) == wrappers[0]
    save_ids, load_ids = [5, 9, 40, 2], [60, 61, 62, 63]
    hashes = sc.make_block_hashes(4, 31)
    expected = [[[bytes(b[off + s * seg: off + (s + 1) * seg]) for off in (0, nb * seg)] for s in save_ids] for b in before]
    job = dict(names=[f"l{i}" for i in range(n_layers)], wrappers=[w.to_bytes() for w in wrappers], device_id=0,
               num_blocks=[nb] * n_layers, bytes_per_block=[seg] * n_layers, kv_stride_bytes=[nb * seg] * n_layers,
               segments=[2] * n_layers, hashes=hashes, save_ids=save_ids, load_ids=load_ids, expected=expected)
    with tempfile.NamedTemporaryFile(suffix=".pkl", delete=False) as f:
        pickle.dump(job, f)
        path = f.name
    try:
        proc = subprocess.run([sys.executable, os.path.join(HERE, "ipc_child.py"), path], stdout=subprocess.PIPE,
                              stderr=subprocess.PIPE, text=True, timeout=300)
    finally:
        os.unlink(path)
    lines = [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]
    assert proc.returncode == 0 and lines, proc.stderr[-3000:]
    out = json.loads(lines[-1])
    assert out["images_ok"], "host images stored by the other process differ from this process's KV bytes"
    assert out["hits"] == 4 and out["load_failures"] == 0
    assert out["save_bytes"] == out["load_bytes"] == n_layers * 4 * 2 * seg
    torch.cuda.synchronize()
    for b, t in zip(before, caches):      # the other process wrote the loaded blocks into this process's memory
        want = b.copy()
        for s, d in zip(save_ids, load_ids):
            for off in (0, nb * seg):
                want[off + d * seg: off + (d + 1) * seg] = b[off + s * seg: off + (s + 1) * seg]
        assert np.array_equal(storage_bytes(t), want)


def test_a_region_cannot_be_opened_by_its_exporter_and_bad_regions_are_rejected():
    import torch

    import pegaflow_b200 as pf
    from pegaflow_b200.ipc import CudaIPCWrapper

    t = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    w = CudaIPCWrapper(t)
    with pytest.raises(pf.PegaFlowError):      # CUDA refuses to map a handle in the process that made it
        w.open()
    with pytest.raises(ValueError, match="zero storage offset"):
        CudaIPCWrapper(t[16:])
