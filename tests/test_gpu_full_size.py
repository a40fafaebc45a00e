"""The Llama-3.1-8B configuration at its full size through the engine API: 32 layers, K and V
regions of 8192 blocks x 32 KiB each (16 GiB of KV cache), 8 requests of 640 scattered blocks
(10 GiB each way).  Too large for the CPU oracle, so the check is a property that needs no
second implementation: after save -> load into other block ids, every destination block holds
exactly what its source block held and every other block of the cache is untouched.  The whole
cache is compared on the GPU with torch, bit for bit.

PEGAFLOW_FULL_SIZE_REQUESTS (default 8, the configuration's count) runs fewer requests for a
quick check; geometry, block ids and code path are the same.
"""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

LAYERS, GPU_BLOCKS, SEG_BYTES, BLOCKS_PER_REQUEST = 32, 8192, 32768, 640


def test_llama31_8b_full_size_round_trip_leaves_every_other_block_untouched():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("this test needs a CUDA device (there is no CPU fallback to test)")
    import pegaflow_b200 as pf

    n_req = int(os.environ.get("PEGAFLOW_FULL_SIZE_REQUESTS", "8"))
    assert 1 <= n_req <= 8
    device = torch.device("cuda", 0)
    gen = torch.Generator(device=device)
    gen.manual_seed(44)
    kv = []
    for _ in range(LAYERS):
        t = torch.empty((2, GPU_BLOCKS, SEG_BYTES // 2), dtype=torch.bfloat16, device=device)
        t.normal_(0.0, 1.0, generator=gen)
        kv.append(t.view(torch.int16))      # bit patterns: NaN-safe equality
    rng = np.random.default_rng(44)
    total = n_req * BLOCKS_PER_REQUEST
    src = rng.permutation(GPU_BLOCKS - 1)[:total] + 1     # id 0 is vLLM's null block
    dst = rng.permutation(GPU_BLOCKS - 1)[:total] + 1
    payload = LAYERS * 2 * total * SEG_BYTES

    # one global pool, so that its whole capacity is usable whatever the host's NUMA layout: a block
    # evicted for lack of room would show up as a prefix miss below
    eng = pf.PegaEngine(payload + (512 << 20), enable_numa_affinity=False)
    try:
        names = [f"model.layers.{l}.self_attn.attn" for l in range(LAYERS)]
        region = 2 * GPU_BLOCKS * SEG_BYTES
        eng.register_context_layer_batch_strided(
            "full", "full-ns", 0, 0, 0, 1, 1, names, [t.data_ptr() for t in kv], [region] * LAYERS,
            [GPU_BLOCKS] * LAYERS, [SEG_BYTES] * LAYERS, [GPU_BLOCKS * SEG_BYTES] * LAYERS, [2] * LAYERS, None, None,
            "direct", False)
        snapshot = [t.clone() for t in kv]
        torch.cuda.synchronize()
        all_hashes = []
        for r in range(n_req):
            ids = src[r * BLOCKS_PER_REQUEST:(r + 1) * BLOCKS_PER_REQUEST].tolist()
            hashes = [b"full%02d" % r + int(i).to_bytes(4, "little") for i in range(BLOCKS_PER_REQUEST)]
            eng.batch_save("full", 0, 0, 0, [(name, ids, hashes) for name in names])
            all_hashes.append(hashes)
        eng.flush_saves()
        pending = []
        for r, hashes in enumerate(all_hashes):
            blocks, missing = eng.query_prefix("full", hashes)
            assert missing == 0 and len(blocks) == BLOCKS_PER_REQUEST
            lease = eng.create_query_lease("full", blocks)
            ids = dst[r * BLOCKS_PER_REQUEST:(r + 1) * BLOCKS_PER_REQUEST].tolist()
            pending.append(eng.batch_load_async("full", 0, 0, [names], [(lease, [ids])]))
        for p in pending:
            assert p.wait(120) == 1, p.error()
        torch.cuda.synchronize()
        m = eng.metrics()
        assert m["save_bytes"] == payload and m["load_bytes"] == payload and m["load_failures"] == 0
        src_idx = torch.from_numpy(src.astype(np.int64)).to(device)
        dst_idx = torch.from_numpy(dst.astype(np.int64)).to(device)
        for l in range(LAYERS):
            want = snapshot[l]
            want[:, dst_idx] = want[:, src_idx]      # the right-hand side is gathered before the scatter
            assert torch.equal(kv[l], want), f"layer {l}: the cache differs from save -> load of the snapshot"
            snapshot[l] = None
    finally:
        eng.close()
