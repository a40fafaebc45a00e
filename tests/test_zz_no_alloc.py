"""The allocation-free save entry point against the oracle and against the regular entry point.

`pf_save_blocks_noalloc` serves callers that cannot allocate device memory when they need blocks
copied out (all free HBM already belongs to the KV cache; cudaMalloc's device-wide synchronisation
is not affordable; a stream capture is running elsewhere).  It stages through an area built into
the library instead of the backend's heap-allocated ring.  Its output must be the bytes the CPU
oracle packs for the same blocks (descriptor pairing of gpu_worker.rs:353-423 executed with
memcpy) and byte-identical to what `pf_backend_save_layers` writes - also on a second call, when
the shared staging area still holds the first call's bytes.  This file sorts last on purpose: a
run that stops at the first failure has then already run every other test."""
import numpy as np
import pytest

from oracle import pf_oracle as po
from tests.gpu_util import CudaMem, host_view

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device (there is no CPU fallback to test)")
    import pegaflow_b200 as pf

    return pf, torch


def _oracle_image(init, num_blocks, seg, n_ranges, ids):
    """What the reference's save leaves on the host for these blocks: range 0 of every block back to
    back, then range 1 (one dense host allocation per range)."""
    shadow = init.copy()
    n = len(ids)
    lay = po.KVCacheLayout(shadow.ctypes.data, shadow.size, num_blocks, seg, num_blocks * seg if n_ranges == 2 else 0,
                           n_ranges)
    out = np.full(n * seg * n_ranges, 0x33, dtype=np.uint8)
    blocks = [(int(b), [po.HostSeg(out.ctypes.data + (r * n + i) * seg, out.ctypes.data + (r * n + i) * seg, r)
                        for r in range(n_ranges)], 0) for i, b in enumerate(ids)]
    descs, nd, total = po.build_copy_descs([(lay, blocks)])
    assert total == out.size
    po.execute(descs, nd, host_is_src=False)
    return out


@pytest.mark.parametrize("n_ranges,seg", [(2, 32768), (1, 73728), (2, 4096), (1, 1001), (2, 1001)])
def test_noalloc_save_matches_the_oracle_and_the_regular_save_twice_in_a_row(env, n_ranges, seg):
    """(2, 1001): the second range starts at an odd offset of the staging area, so its gather takes
    the byte path."""
    pf, torch = env
    mem = CudaMem(0)
    rng = np.random.default_rng(n_ranges * 1000 + seg)
    num_blocks = 96
    kv_stride = num_blocks * seg if n_ranges == 2 else 0
    dev = mem.alloc(num_blocks * seg * n_ranges)
    init = rng.integers(0, 256, size=dev.numel(), dtype=np.uint8)
    mem.write(dev, init)
    layout = (dev.data_ptr(), seg, kv_stride, seg, n_ranges, num_blocks)
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
            assert np.array_equal(host_view(got_h, total), _oracle_image(init, num_blocks, seg, n_ranges, ids)), \
                f"call {call}: differs from the oracle"
            assert np.array_equal(host_view(got_h, total), host_view(want_h, total)), \
                f"call {call}: differs from pf_backend_save_layers"
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
        pf.save_blocks_noalloc(0, (dev.data_ptr(), 4096, 0, 4096, 1), [], host, 0)   # empty batch is a no-op
        too_many = list(range(4)) * ((pf._native.NOALLOC_MAX_BLOCKS // 4) + 1)
        with pytest.raises(pf.PegaflowInvalidArgument, match="limit of 16384 blocks"):
            pf.save_blocks_noalloc(0, (dev.data_ptr(), 16, 0, 16, 1), too_many, host, 16 << 20)
        with pytest.raises(pf.PegaflowInvalidArgument, match="exceed the built-in staging area"):
            pf.save_blocks_noalloc(0, (dev.data_ptr(), 65536, 0, 65536, 1), [0] * 129, host, 16 << 20)
        with pytest.raises(pf.PegaflowInvalidArgument, match="destination holds"):
            pf.save_blocks_noalloc(0, (dev.data_ptr(), 4096, 0, 4096, 1), [0, 1], host, 4096)
        # a cache of 256 blocks of 4 KiB: id 256 lies outside it and nothing may be launched for it
        host_view(host, 8192)[:] = 0x5A
        with pytest.raises(pf.PegaflowInvalidArgument, match="block_id 256 out of range"):
            pf.save_blocks_noalloc(0, (dev.data_ptr(), 4096, 0, 4096, 1, 256), [3, 256], host, 8192)
        torch.cuda.synchronize()
        assert (host_view(host, 8192) == 0x5A).all(), "a rejected call must not have written anything"
    finally:
        pool.close()
