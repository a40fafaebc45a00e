"""The allocation-free save entry point against the regular one.

`pf_save_blocks_noalloc` serves callers that cannot allocate device memory when they need blocks
copied out (all free HBM already belongs to the KV cache; cudaMalloc's device-wide synchronisation
is not affordable; a stream capture is running elsewhere).  It stages through an area built into
the library instead of the backend's heap-allocated ring, so its output must be byte-identical to
`pf_backend_save_layers` for the same blocks - also on a second call, when the shared staging area
still holds the first call's bytes.  This file sorts last on purpose: a run that stops at the first
failure has then already run every other test."""
import numpy as np
import pytest

from tests.gpu_util import CudaMem, host_view

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device (there is no CPU fallback to test)")
    import pegaflow_b200 as pf

    return pf, torch


@pytest.mark.parametrize("n_ranges,seg", [(2, 32768), (1, 73728), (2, 4096), (1, 1001)])
def test_noalloc_save_matches_regular_save_twice_in_a_row(env, n_ranges, seg):
    pf, torch = env
    mem = CudaMem(0)
    rng = np.random.default_rng(n_ranges * 1000 + seg)
    num_blocks = 96
    kv_stride = num_blocks * seg if n_ranges == 2 else 0
    dev = mem.alloc(num_blocks * seg * n_ranges)
    mem.write(dev, rng.integers(0, 256, size=dev.numel(), dtype=np.uint8))
    layout = (dev.data_ptr(), seg, kv_stride, seg, n_ranges)
    pool = pf.PinnedPool(64 << 20)
    be = pf.TransferBackend(0, min_dma_bytes=64 << 10)
    stream = torch.cuda.Stream()
    try:
        for call, n in enumerate((40, 17)):      # second call: fewer, different blocks
            ids = rng.permutation(num_blocks)[:n].tolist()
            total = n * seg * n_ranges
            want_h, want_d, h1 = pool.alloc(total)
            got_h, got_d, h2 = pool.alloc(total)
            host_view(want_h, total)[:] = 0x11
            host_view(got_h, total)[:] = 0x22
            runs = [[pf.HostRun(0, n, want_h + r * n * seg, want_d + r * n * seg, seg)] for r in range(n_ranges)]
            be.save_layers([pf.LayerXfer(dev.data_ptr(), seg, kv_stride, seg, n_ranges, ids, runs)], stream.cuda_stream)
            pf.save_blocks_noalloc(0, layout, ids, got_h, total, stream.cuda_stream)
            stream.synchronize()
            assert np.array_equal(host_view(got_h, total), host_view(want_h, total)), f"call {call} differs"
            pool.release(h1)
            pool.release(h2)
    finally:
        be.close()
        pool.close()


def test_noalloc_limits_are_rejected_with_a_clear_error(env):
    pf, torch = env
    mem = CudaMem(0)
    dev = mem.alloc(1 << 20)
    pool = pf.PinnedPool(32 << 20)
    host, _, _ = pool.alloc(16 << 20)
    try:
        too_many = list(range(4)) * ((pf._native.NOALLOC_MAX_BLOCKS // 4) + 1)
        with pytest.raises(pf.PegaflowInvalidArgument, match="limit of 16384 blocks"):
            pf.save_blocks_noalloc(0, (dev.data_ptr(), 16, 0, 16, 1), too_many, host, 16 << 20)
        with pytest.raises(pf.PegaflowInvalidArgument, match="exceed the built-in staging area"):
            pf.save_blocks_noalloc(0, (dev.data_ptr(), 65536, 0, 65536, 1), [0] * 129, host, 16 << 20)
        with pytest.raises(pf.PegaflowInvalidArgument, match="destination holds"):
            pf.save_blocks_noalloc(0, (dev.data_ptr(), 4096, 0, 4096, 1), [0, 1], host, 4096)
        pf.save_blocks_noalloc(0, (dev.data_ptr(), 4096, 0, 4096, 1), [], host, 0)   # empty batch is a no-op
    finally:
        pool.close()
