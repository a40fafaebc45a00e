"""Several caller threads on one engine at once — saves, prefix queries, leases, loads — with a
pool small enough that every save evicts someone's blocks.  The rules under test: a lease pins its
blocks' bytes (storage/read_cache.rs:362-389), evicted blocks simply stop hitting, and whatever a
load delivers is byte for byte what was saved under those hashes."""
import threading

import numpy as np
import pytest

from tests import scenarios as sc
from tests.gpu_util import CudaMem

pytestmark = pytest.mark.gpu


def test_concurrent_callers_under_eviction_pressure():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("this test needs a CUDA device")
    import pegaflow_b200 as pf

    n_threads, per_thread, seg, n_layers, rounds = 4, 128, 16384, 3, 30
    num_blocks = n_threads * per_thread * 2            # each thread: its own source blocks and destination blocks
    eng = pf.PegaEngine(24 << 20, min_dma_bytes=64 << 10)     # holds half of the 48 MiB of distinct blocks
    mem = CudaMem(0)
    try:
        layers = [sc.Layer(f"l{i}", num_blocks, seg, segments=2, kv_stride=num_blocks * seg) for i in range(n_layers)]
        sc.register(eng, mem, "stress", "ns", layers)
        fills = [sc.seeded_bytes(L.region_bytes, 500 + i) for i, L in enumerate(layers)]
        for L, f in zip(layers, fills):
            mem.write(L.buf, f)
        mem.sync()
        names = [L.name for L in layers]
        errors, stats = [], {"loads": 0, "hit_blocks": 0, "misses": 0}
        lock = threading.Lock()

        def caller(t):
            try:
                torch.cuda.set_device(0)
                rng = np.random.default_rng(900 + t)
                src0, dst0 = t * 2 * per_thread, t * 2 * per_thread + per_thread
                for r in range(rounds):
                    n = int(rng.integers(4, 17))
                    src = (src0 + rng.permutation(per_thread)[:n]).tolist()
                    # a block's hash is a function of the block: the same bytes are always stored under it
                    hashes = [b"stress-%04d" % b for b in src]
                    try:
                        eng.batch_save("stress", 0, 0, 0, [(name, src, hashes) for name in names])
                    except pf.PegaflowInternal as e:
                        # every evictable block may be pinned by the other threads' leases for a moment
                        if "pinned pool exhausted" not in str(e):
                            raise
                        with lock:
                            stats["exhausted"] = stats.get("exhausted", 0) + 1
                        continue
                    eng.flush_saves()
                    blocks, _missing = eng.query_prefix("stress", hashes)
                    hit = len(blocks)
                    with lock:
                        stats["hit_blocks"] += hit
                        stats["misses"] += n - hit
                    if hit == 0:
                        continue
                    lease = eng.create_query_lease("stress", blocks)
                    del blocks
                    dst = (dst0 + rng.permutation(per_thread)[:hit]).tolist()
                    done = eng.batch_load_async("stress", 0, 0, [names], [(lease, [dst])])
                    if done.wait(30) != 1:
                        raise RuntimeError("load failed: " + done.error())
                    for L, f in zip(layers, fills):
                        got = L.buf.view(2, num_blocks, seg)[:, torch.tensor(dst, device=L.buf.device)].cpu().numpy()
                        want = f.reshape(2, num_blocks, seg)[:, src[:hit]]
                        if not np.array_equal(got, want):
                            raise AssertionError(f"thread {t} round {r}: loaded bytes differ from the saved ones")
                    with lock:
                        stats["loads"] += 1
            except Exception as e:       # reported by the main thread
                errors.append(e)

        threads = [threading.Thread(target=caller, args=(t,)) for t in range(n_threads)]
        for th in threads:
            th.start()
        for th in threads:
            th.join(120)
        assert not any(th.is_alive() for th in threads), "a caller thread is stuck"
        assert not errors, errors[:2]
        m = eng.metrics()
        assert stats["loads"] > n_threads * rounds // 2 and m["load_failures"] == 0, (stats, m)
        assert m["evicted_blocks"] > 0, "the pool was meant to be too small"
    finally:
        eng.close()
