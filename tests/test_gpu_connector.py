"""The worker-connector mirror on a GPU: registration inferred from real tensors in vLLM's cache
shapes (FlashAttention KV-first, HND strides, FlashInfer interleaved, MLA latent with 64->128
virtual blocks, cross-layer fused buffer), batched and layer-wise saves, load with per-layer waits."""
import time

import numpy as np
import pytest

from tests import scenarios as sc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device (there is no CPU fallback to test)")
    import pegaflow_b200 as pf
    from pegaflow_b200 import connector

    return pf, connector, torch


def _wait_loads(conn, want, timeout=10):
    done, failed, deadline = [], [], time.time() + timeout
    while len(done) + len(failed) < want and time.time() < deadline:
        d, f = conn.get_finished()
        done += d
        failed += f
        time.sleep(0.001)
    return done, failed


SHAPES = {
    # name: (builder(torch, device) -> tensor, block_size, is_mla, expect (layout, segments, num_blocks))
    "flash_attn_nhd": (lambda t, d: t.empty((2, 48, 16, 8, 128), dtype=t.bfloat16, device=d), 16, False,
                       ("KV-first", 2, 48)),
    "flash_attn_hnd": (lambda t, d: t.empty((2, 48, 8, 16, 128), dtype=t.bfloat16, device=d).permute(0, 1, 3, 2, 4),
                       16, False, ("KV-first", 2, 48)),
    "flashinfer_interleaved": (lambda t, d: t.empty((48, 2, 16, 8, 128), dtype=t.bfloat16, device=d), 16, False,
                               ("blocks-first", 1, 48)),
    "mla_latent_bf16": (lambda t, d: t.empty((48, 64, 576), dtype=t.bfloat16, device=d), 64, True,
                        ("blocks-first", 1, 48)),
    "mla_latent_fp8_virtual_blocks": (lambda t, d: t.empty((48, 64, 576), dtype=t.uint8, device=d), 128, True,
                                      ("blocks-first", 1, 24)),
    "cross_layer_fused": (lambda t, d: t.empty((48, 6, 2, 16, 2, 128), dtype=t.bfloat16, device=d), 16, False,
                          ("blocks-first", 1, 48)),
}


@pytest.mark.parametrize("name", list(SHAPES))
def test_register_save_load_in_vllm_cache_shapes(env, name):
    pf, connector, torch = env
    build, block_size, is_mla, (layout, segments, num_blocks) = SHAPES[name]
    dev = torch.device("cuda", 0)
    eng = pf.PegaEngine(256 << 20, min_dma_bytes=64 << 10)
    try:
        conn = connector.PegaWorkerConnector(connector.InProcEngineClient(eng), eng, instance_id="c", namespace="ns",
                                             device_id=0, block_size=block_size, is_mla=is_mla)
        n_layers = 1 if name == "cross_layer_fused" else 3
        caches = {}
        for i in range(n_layers):
            t = build(torch, dev)
            base = t if t.is_contiguous() else t.permute(0, 1, 3, 2, 4)   # the HND view's storage order
            base.view(torch.uint8).random_(0, 256, generator=torch.Generator(device=dev).manual_seed(7 + i))
            caches[f"model.layers.{i}.attn"] = t
        if name == "cross_layer_fused":
            conn.register_cross_layers_kv_cache(next(iter(caches.values())))
            caches = {conn.registered_layers[0]: next(iter(caches.values()))}
            assert conn.registered_layers == ["ALL_LAYERS"]
        else:
            conn.register_kv_caches(caches)
        info = next(iter(conn.registrations.values()))
        assert (info.layout, info.segments, info.num_blocks) == (layout, segments, num_blocks)
        rng = np.random.default_rng(5)
        src = (rng.permutation(num_blocks - 1)[:8] + 1).tolist()
        dst = (rng.permutation(num_blocks - 1)[:8] + 1).tolist()
        hashes = sc.make_block_hashes(8, 3)

        def storage_bytes(t):
            return torch.empty(0, dtype=torch.uint8, device=dev).set_(t.untyped_storage()).clone()

        before = {k: storage_bytes(t) for k, t in caches.items()}
        conn.wait_for_save([(k, [0] + src, [b"null"] + hashes) for k in caches])   # id 0 is skipped
        q = conn.client.query_prefetch("c", hashes, "req-1")
        assert q.num_hit_blocks == 8 and q.hit_positions == list(range(8))
        assert conn.client.query_prefetch("c", [b"null"], "req-0").num_hit_blocks == 0
        for t in caches.values():
            torch.empty(0, dtype=torch.uint8, device=dev).set_(t.untyped_storage()).zero_()
        conn.start_load_kv([("req-1", q.lease, dst)])
        stream = torch.cuda.Stream()
        for k in caches:
            conn.wait_for_layer_load(k, stream.cuda_stream)
        stream.synchronize()   # every layer's event has fired, so all bytes have landed
        ratio = info.physical_blocks_per_logical_block
        for k, t in caches.items():
            got = storage_bytes(t)
            want = torch.zeros_like(got)
            if info.segments == 2:
                seg, kv = info.bytes_per_block, info.kv_stride_bytes
                for s, d_ in zip(src, dst):
                    for off in (0, kv):
                        want[off + d_ * seg: off + (d_ + 1) * seg] = before[k][off + s * seg: off + (s + 1) * seg]
            else:
                bb = info.bytes_per_block
                for s, d_ in zip(src, dst):
                    want[d_ * bb:(d_ + 1) * bb] = before[k][s * bb:(s + 1) * bb]
            assert torch.equal(got, want), f"{k}: bytes differ (ratio {ratio})"
        done, failed = _wait_loads(conn, 1)
        assert done == ["req-1"] and not failed and not conn.get_block_ids_with_load_errors()
    finally:
        eng.close()


def test_layerwise_saves_and_failed_load_reporting(env):
    pf, connector, torch = env
    dev = torch.device("cuda", 0)
    eng = pf.PegaEngine(128 << 20, min_dma_bytes=64 << 10)
    try:
        conn = connector.PegaWorkerConnector(connector.InProcEngineClient(eng), eng, instance_id="lw", namespace="ns",
                                             device_id=0, block_size=16)
        caches = {f"l{i}": torch.empty((2, 32, 16, 2, 128), dtype=torch.bfloat16, device=dev) for i in range(4)}
        conn.register_kv_caches(caches)
        compute = torch.cuda.Stream()
        hashes = sc.make_block_hashes(6, 9)
        ids = [3, 9, 1, 30, 12, 7]
        events = []
        for i, (k, t) in enumerate(caches.items()):
            with torch.cuda.stream(compute):
                t.view(torch.uint8).random_(0, 256)      # the layer's forward pass writing its KV
                ev = torch.cuda.Event()
                ev.record(compute)
            events.append(ev)
            conn.save_kv_layer(k, ids, hashes, ev.cuda_event)
        conn.wait_for_save()
        q = conn.client.query_prefetch("lw", hashes, "r")
        assert q.num_hit_blocks == 6
        snap = {k: t.clone() for k, t in caches.items()}
        conn.start_load_kv([("r", q.lease, [20, 21, 22, 23, 24, 25])])
        done, failed = _wait_loads(conn, 1)
        assert done == ["r"]
        for k, t in caches.items():
            # compare bytes: random bf16 bit patterns contain NaNs
            assert torch.equal(t[:, 20:26].contiguous().view(torch.uint8),
                               snap[k][:, ids].contiguous().view(torch.uint8))
        # a load with an unknown lease is reported, not raised (worker.py:650-684, 729-739)
        conn.start_load_kv([("bad", b"\7" * 16, [1, 2])])
        assert conn.get_block_ids_with_load_errors() == {1, 2}
        # a destination out of range is rejected before anything is enqueued; the blocks are reported
        q2 = conn.client.query_prefetch("lw", hashes, "r2")
        conn.start_load_kv([("r2", q2.lease, [20, 21, 22, 23, 24, 99])])
        assert 99 in conn.get_block_ids_with_load_errors()
        assert eng.metrics()["load_failures"] == 0
    finally:
        eng.close()


def test_scheduler_and_worker_connectors_end_to_end(env):
    """A cold request and a warm one through both halves of the connector and the engine: the
    scheduler plans saves as blocks fill, the worker stores them; the second request's lookup hits,
    its load intent carries the lease, and the worker's load puts the first request's bytes into the
    second request's blocks."""
    pf, connector, torch = env
    from types import SimpleNamespace as NS

    from pegaflow_b200.scheduler import SchedulerConnector

    dev = torch.device("cuda", 0)
    eng = pf.PegaEngine(256 << 20, min_dma_bytes=64 << 10)
    try:
        client = connector.InProcEngineClient(eng)
        worker = connector.PegaWorkerConnector(client, eng, instance_id="both", namespace="ns", device_id=0, block_size=16)
        sched = SchedulerConnector([client], instance_id="both", block_size=16)
        caches = {f"l{i}": torch.empty((2, 64, 16, 2, 128), dtype=torch.bfloat16, device=dev) for i in range(3)}
        for i, t in enumerate(caches.values()):
            t.view(torch.uint8).random_(0, 256, generator=torch.Generator(device=dev).manual_seed(40 + i))
        worker.register_kv_caches(caches)
        hashes = sc.make_block_hashes(5, 12)

        def request(name, n_tokens):
            return NS(request_id=name, block_hashes=list(hashes[:n_tokens // 16]), num_tokens=n_tokens)

        def step(new=(), running=()):
            return NS(scheduled_new_reqs=[NS(req_id=r, block_ids=([*ids],), num_computed_tokens=c) for r, ids, c, _ in new],
                      scheduled_cached_reqs=NS(req_ids=[r for r, *_ in running], new_block_ids=[None for _ in running],
                                               num_computed_tokens=[c for _, c, _ in running], resumed_req_ids=set()),
                      num_scheduled_tokens={**{r: n for r, _, _, n in new}, **{r: n for r, _, n in running}},
                      preempted_req_ids=set())

        # cold: 80-token prompt in blocks 10..14, prefilled in two chunks
        cold = request("cold", 80)
        assert sched.get_num_new_matched_tokens(cold, 0) == (0, False)
        sched.update_state_after_alloc(cold, NS(get_block_ids=lambda: ([10, 11, 12, 13, 14],), blocks=[[]]), 0)
        meta = sched.build_connector_meta(step(new=[("cold", [10, 11, 12, 13, 14], 0, 48)]))
        assert list(meta.save_intents["cold"].block_ids_by_group[0]) == [10, 11, 12]
        sent = worker.wait_for_save_from_metadata(meta)
        meta = sched.build_connector_meta(step(running=[("cold", 48, 32)]))
        assert list(meta.save_intents["cold"].block_ids_by_group[0]) == [13, 14]
        sent |= worker.wait_for_save_from_metadata(meta)
        assert sched.request_finished(cold, ([10, 11, 12, 13, 14],)) == (True, None)
        sched.update_connector_output(NS(finished_sending=sent, finished_recving=None))
        assert sched.request_finished(cold, ([10, 11, 12, 13, 14],)) == (False, None)

        # warm: the same prompt; one token is left to compute, the other 79 come from the pool
        warm = request("warm", 80)
        tokens, load_async = sched.get_num_new_matched_tokens(warm, 0)
        assert (tokens, load_async) == (79, True)
        dst = [30, 31, 32, 33, 34]
        blocks = NS(get_block_ids=lambda: (dst,), blocks=[[NS(block_hash=None) for _ in dst]])
        sched.update_state_after_alloc(warm, blocks, tokens)
        meta = sched.build_connector_meta(step(new=[("warm", dst, 79, 1)]))
        assert list(meta.load_intents["warm"].block_ids_by_group[0]) == dst and not meta.save_intents
        before = {k: t.clone() for k, t in caches.items()}
        worker.start_load_kv_from_metadata(meta)
        done, failed = _wait_loads(worker, 1)
        assert done == ["warm"] and not failed
        torch.cuda.synchronize()
        for k, t in caches.items():
            assert torch.equal(t[:, dst].view(torch.uint8), before[k][:, [10, 11, 12, 13, 14]].view(torch.uint8))
        assert eng.metrics()["load_failures"] == 0
    finally:
        eng.close()
