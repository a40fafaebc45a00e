"""Parity of the CUDA transfer backend with the CPU oracle, through the C ABI.

Bit-exact is the bar: this is byte movement.  The oracle executes the same descriptor batch
with memcpy (oracle/pf_oracle.c: pfo_build_copy_descs + pfo_execute)."""
import numpy as np
import pytest

from oracle import pf_oracle as po
from tests.gpu_util import CudaMem, host_view, make_event

pytestmark = pytest.mark.gpu

ROUTES = {"auto": 0, "staged": 1, "zerocopy": 2}


@pytest.fixture(scope="module")
def env():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device (there is no CPU fallback to test)")
    import pegaflow_b200 as pf

    mem = CudaMem(0)
    pool = pf.PinnedPool(256 << 20)
    yield pf, mem, pool, torch
    pool.close()


def _pattern(n):
    return ((np.arange(n, dtype=np.uint64) * 31 + 7) & 0xFF).astype(np.uint8)


@pytest.mark.parametrize("route", list(ROUTES))
def test_kernel_matches_pattern_both_directions(env, kats, route):
    """The reference's own backend test (transfer/kernel.rs:205-267): 257 segments of 4112 bytes."""
    pf, mem, pool, torch = env
    k = kats["kernel_roundtrip"]
    n, seg = k["segments"], k["segment_bytes"]
    total = n * seg
    host, host_dev, handle = pool.alloc(total)
    hv = host_view(host, total)
    dev = mem.alloc(total)
    pattern = _pattern(total)
    be = pf.TransferBackend(0, route=ROUTES[route], min_dma_bytes=64 << 10)
    descs, nd = be.make_descs((dev.data_ptr() + i * seg, host + i * seg, host_dev + i * seg, seg) for i in range(n))
    stream = torch.cuda.Stream()
    hv[:] = pattern
    be.h2d(descs, nd, stream.cuda_stream)
    stream.synchronize()
    assert np.array_equal(mem.read(dev), pattern)
    hv[:] = 0
    be.d2h(descs, nd, stream.cuda_stream)
    stream.synchronize()
    assert np.array_equal(hv, pattern)
    st = be.stats()
    assert st["device_status"] == 0
    if route == "zerocopy":
        assert st["bytes_zero_copy"] == 2 * total and st["dma_copies"] == 0 and st["kernel_launches"] > 0
    else:
        # contiguous on both sides: one plain DMA per direction, nothing to gather (memcpy.rs:25-55)
        assert st["bytes_staged"] == 2 * total and st["dma_copies"] == 2 and st["kernel_launches"] == 0
    be.close()
    pool.release(handle)


@pytest.mark.parametrize("route", list(ROUTES))
@pytest.mark.parametrize("layout", ["contiguous", "strided_device", "shuffled", "shuffled_with_a_gap", "reversed"])
def test_descriptor_batches_in_the_reference_bench_layouts(env, route, layout):
    """The fragment layouts of the reference's transfer bench (benches/transfer_h2d.rs:62-103) and two
    more orders, against the oracle's memcpy execution of the same descriptors, both directions."""
    pf, mem, pool, torch = env
    n, seg = 1500, 4096
    rng = np.random.default_rng(21)
    slots = np.arange(n)
    if layout == "contiguous":
        d_slots, h_slots = slots, slots
    elif layout == "strided_device":
        d_slots, h_slots = slots * 2, slots
    elif layout == "reversed":
        d_slots, h_slots = slots[::-1] * 2, slots[::-1]
    else:
        p = rng.permutation(n)
        d_slots, h_slots = p, p
        if layout == "shuffled_with_a_gap":
            h_slots = np.where(p >= 700, p + 1, p)     # the host range is not dense: slot 700 stays untouched
    dev_bytes, host_bytes = (int(d_slots.max()) + 1) * seg, (int(h_slots.max()) + 1) * seg
    host, host_dev, handle = pool.alloc(host_bytes)
    hv = host_view(host, host_bytes)
    dev = mem.alloc(dev_bytes)
    be = pf.TransferBackend(0, route=ROUTES[route], min_dma_bytes=64 << 10)
    copies = [(dev.data_ptr() + int(d) * seg, host + int(h) * seg, host_dev + int(h) * seg, seg) for d, h in zip(d_slots, h_slots)]
    descs, nd = be.make_descs(copies)
    stream = torch.cuda.Stream()
    # host -> device
    hv[:] = rng.integers(0, 256, size=host_bytes, dtype=np.uint8)
    mem.zero(dev)
    be.h2d(descs, nd, stream.cuda_stream)
    stream.synchronize()
    want = np.zeros(dev_bytes, dtype=np.uint8)
    for d, h in zip(d_slots, h_slots):
        want[int(d) * seg:(int(d) + 1) * seg] = hv[int(h) * seg:(int(h) + 1) * seg]
    assert np.array_equal(mem.read(dev), want)
    # device -> host
    fresh = rng.integers(0, 256, size=dev_bytes, dtype=np.uint8)
    mem.write(dev, fresh)
    hv[:] = 0
    be.d2h(descs, nd, stream.cuda_stream)
    stream.synchronize()
    want_host = np.zeros(host_bytes, dtype=np.uint8)
    for d, h in zip(d_slots, h_slots):
        want_host[int(h) * seg:(int(h) + 1) * seg] = fresh[int(d) * seg:(int(d) + 1) * seg]
    assert np.array_equal(hv, want_host)
    st = be.stats()
    assert st["device_status"] == 0 and st["bytes_staged"] + st["bytes_zero_copy"] == 2 * n * seg
    if route != "zerocopy" and layout in ("shuffled", "reversed"):
        assert st["bytes_zero_copy"] == 0, "a dense host range in any descriptor order takes the staged route"
    be.close()
    pool.release(handle)


@pytest.mark.parametrize("route", ["auto", "zerocopy"])
def test_unaligned_and_ragged_descriptors(env, route):
    """Odd sizes and odd addresses (the reference's kernel falls back to a byte loop,
    kernel.rs:38-43); zero-sized descriptors; descriptors of very different sizes."""
    pf, mem, pool, torch = env
    rng = np.random.default_rng(11)
    sizes = [0, 1, 15, 16, 17, 4111, 4112, 65537, 3, 1 << 20, 31, 100003]
    total_host = sum(sizes) + 64 * len(sizes)
    host, host_dev, handle = pool.alloc(total_host)
    hv = host_view(host, total_host)
    dev = mem.alloc(total_host + 4096)
    dev_init = rng.integers(0, 256, size=dev.numel(), dtype=np.uint8)
    copies, o_descs = [], (po.CopyDesc * len(sizes))()
    shadow = dev_init.copy()
    cur_h, cur_d = 0, 0
    for i, sz in enumerate(sizes):
        cur_h += (i * 7) % 13 + 1   # odd, mutually different misalignment on both sides
        cur_d += (i * 5) % 11 + 2
        copies.append((dev.data_ptr() + cur_d, host + cur_h, host_dev + cur_h, sz))
        o_descs[i] = po.CopyDesc(shadow.ctypes.data + cur_d, 0, 0, sz, 0, 0)
        cur_h += sz
        cur_d += sz
    be = pf.TransferBackend(0, route=ROUTES[route])
    descs, nd = be.make_descs(copies)
    # device -> host
    mem.write(dev, dev_init)
    hv[:] = 0xEE
    want_host = np.full(total_host, 0xEE, dtype=np.uint8)
    for i in range(nd):
        o_descs[i].host = want_host.ctypes.data + (copies[i][1] - host)
    po.execute(o_descs, nd, host_is_src=False)
    be.d2h(descs, nd, 0)
    mem.sync()
    assert np.array_equal(hv, want_host)
    # host -> device
    hv[:] = rng.integers(0, 256, size=total_host, dtype=np.uint8)
    host_copy = hv.copy()
    for i in range(nd):
        o_descs[i].host = host_copy.ctypes.data + (copies[i][1] - host)
    po.execute(o_descs, nd, host_is_src=True)
    be.h2d(descs, nd, 0)
    mem.sync()
    assert np.array_equal(mem.read(dev), shadow)
    assert be.stats()["device_status"] == 0
    be.close()
    pool.release(handle)


def _layer_case(name, num_blocks, seg, segments, kv_stride, block_stride, n_move, host_stride_pad, seed,
                consecutive=False):
    return dict(name=name, num_blocks=num_blocks, seg=seg, segments=segments, kv_stride=kv_stride,
                block_stride=block_stride, n_move=n_move, pad=host_stride_pad, seed=seed, consecutive=consecutive)


LAYER_CASES = [
    # Qwen3-0.6B-like: K and V regions, NHD, 32 KiB segments
    _layer_case("kv_split_32k", 64, 32768, 2, 64 * 32768, 0, 17, 0, 1),
    # interleaved K/V (FlashInfer form): collapses to one contiguous 64 KiB block
    _layer_case("interleaved", 32, 32768, 2, 32768, 0, 9, 0, 2),
    # TP8 shard: 4 KiB segments, many blocks
    _layer_case("kv_split_4k", 512, 4096, 2, 512 * 4096, 0, 300, 0, 3),
    # MLA latent, block 64 x 576 bf16, single segment
    _layer_case("mla_bf16", 24, 73728, 1, 0, 0, 11, 0, 4),
    # MLA fp8
    _layer_case("mla_fp8", 24, 36864, 1, 0, 0, 24, 0, 5),
    # one layer inside a cross-layer fused buffer: stride larger than the block
    _layer_case("fused_stride", 16, 8192, 1, 0, 3 * 8192, 16, 0, 6),
    # host stride padded past the segment (the reference's 512-byte rule): 8848 -> 9216
    _layer_case("padded_host", 20, 8848, 2, 20 * 8848 + 48, 0, 13, 368, 7),
    # odd sizes: not a multiple of 16
    _layer_case("odd_bytes", 10, 1001, 1, 0, 0, 7, 0, 8),
    # a single block
    _layer_case("single", 4, 65536, 1, 0, 0, 1, 0, 9),
    # small items that share a kernel chunk: 33 vectors per item, ragged last chunk
    _layer_case("small_528", 700, 528, 2, 700 * 528, 0, 611, 0, 10),
    # small items with a device stride that is not 16-byte aligned: one item per chunk, byte path
    _layer_case("small_unaligned_stride", 300, 2048, 1, 0, 2052, 257, 0, 11),
    # consecutive block ids (a fresh prompt on an ordered free list): one DMA per range, no gather
    _layer_case("consecutive_ids_32k", 64, 32768, 2, 64 * 32768, 0, 20, 0, 12, consecutive=True),
    # consecutive ids, block stride larger than the block and a padded host stride: pitched DMA
    _layer_case("consecutive_ids_pitched", 40, 73728, 1, 0, 2 * 73728, 12, 512, 13, consecutive=True),
    # consecutive ids but short padded rows: stays on the gather route
    _layer_case("consecutive_ids_short_rows", 300, 4096, 2, 300 * 4096, 0, 200, 512, 14, consecutive=True),
]


def _random_layer_cases(count, seed):
    """Seeded random geometries on top of the named ones: segment sizes that are and are not multiples of 16,
    K/V split and interleaved, block strides wider than the block (aligned or not), padded host strides, few and
    many blocks, scattered and consecutive ids.  Geometries the layout rules refuse are drawn again."""
    rng = np.random.default_rng(seed)
    sizes = [16, 48, 528, 1001, 2048, 4096, 4112, 8848, 9216, 32768, 36864, 73728, 100000]
    out = []
    while len(out) < count:
        segments = int(rng.integers(1, 3))
        seg = int(rng.choice(sizes))
        num_blocks = int(rng.choice([2, 3, 17, 64, 300, 600]))
        if num_blocks * seg * segments > 48 << 20:
            continue
        split = segments == 2 and rng.random() < 0.7
        kv_stride = (num_blocks * seg + int(rng.choice([0, 0, 48, 4096]))) if split else (seg if segments == 2 else 0)
        block = seg if split else seg * segments
        block_stride = 0 if rng.random() < 0.6 else block + int(rng.choice([16, 4, 1, block, 512]))
        if split and block_stride:
            kv_stride = (num_blocks - 1) * block_stride + seg + int(rng.choice([0, 64]))
        n_move = int(rng.integers(1, num_blocks + 1))
        case = _layer_case(f"random_{len(out)}_seg{seg}x{segments}_nb{num_blocks}", num_blocks, seg, segments, kv_stride,
                           block_stride, n_move, int(rng.choice([0, 0, 16, 368, 512, 3])), 100 + len(out),
                           consecutive=bool(rng.random() < 0.25))
        try:
            lay = po.KVCacheLayout(0x10000, 1 << 40, num_blocks, seg, kv_stride, segments)
            if block_stride:
                lay.with_block_stride(block_stride)
        except Exception:
            continue
        out.append(case)
    return out


LAYER_CASES += _random_layer_cases(24, 2024)


@pytest.mark.parametrize("route", list(ROUTES))
@pytest.mark.parametrize("case", LAYER_CASES, ids=[c["name"] for c in LAYER_CASES])
def test_layer_save_load_matches_oracle(env, case, route):
    pf, mem, pool, torch = env
    rng = np.random.default_rng(case["seed"])
    lay = po.KVCacheLayout(0x10000, 1 << 40, case["num_blocks"], case["seg"], case["kv_stride"], case["segments"])
    if case["block_stride"]:
        lay.with_block_stride(case["block_stride"])
    n_ranges = 2 if lay.is_split else 1
    range_bytes = case["seg"] if lay.is_split else case["seg"] * case["segments"]
    stride = lay.c.block_stride_bytes
    kv = lay.c.kv_stride_bytes if lay.is_split else 0
    region = (case["num_blocks"] - 1) * stride + range_bytes + kv
    dev = mem.alloc(region)
    init = rng.integers(0, 256, size=region, dtype=np.uint8)
    mem.write(dev, init)
    n = case["n_move"]
    save_ids = rng.permutation(case["num_blocks"])[:n]
    load_ids = rng.permutation(case["num_blocks"])[:n]
    if case["consecutive"]:
        save_ids = int(rng.integers(0, case["num_blocks"] - n + 1)) + np.arange(n)
        load_ids = int(rng.integers(0, case["num_blocks"] - n + 1)) + np.arange(n)
    hstride = range_bytes + case["pad"]
    allocs = [pool.alloc(hstride * n) for _ in range(n_ranges)]
    for a in allocs:
        host_view(a[0], hstride * n)[:] = 0xA5
    runs = [[pf.HostRun(0, n, a[0], a[1], hstride)] for a in allocs]
    be = pf.TransferBackend(0, route=ROUTES[route], min_dma_bytes=64 << 10, staging_slot_bytes=1 << 20)
    stream = torch.cuda.Stream()
    ev = make_event(torch)
    X = pf.LayerXfer(dev.data_ptr(), stride, kv, range_bytes, n_ranges, list(save_ids), runs)
    be.save_layers([X], stream.cuda_stream, [ev.cuda_event])
    ev.synchronize()   # the per-layer event alone must cover the layer's bytes
    # oracle: same layer over numpy memory
    shadow = init.copy()
    olay = po.KVCacheLayout(shadow.ctypes.data, region, case["num_blocks"], case["seg"], case["kv_stride"],
                            case["segments"])
    if case["block_stride"]:
        olay.with_block_stride(case["block_stride"])
    ohost = [np.full(hstride * n, 0xA5, dtype=np.uint8) for _ in range(n_ranges)]

    def blocks(ids):
        return [(int(b), [po.HostSeg(h.ctypes.data + i * hstride, h.ctypes.data + i * hstride, r)
                          for r, h in enumerate(ohost)], 0) for i, b in enumerate(ids)]

    d, nd, total = po.build_copy_descs([(olay, blocks(save_ids))])
    assert total == n * range_bytes * n_ranges
    po.execute(d, nd, host_is_src=False)
    for a, h in zip(allocs, ohost):
        assert np.array_equal(host_view(a[0], hstride * n), h), "host image differs (padding must stay untouched)"
    # load into other block ids
    mem.zero(dev)
    shadow[:] = 0
    X2 = pf.LayerXfer(dev.data_ptr(), stride, kv, range_bytes, n_ranges, list(load_ids), runs)
    be.load_layers([X2], stream.cuda_stream, [ev.cuda_event])
    ev.synchronize()
    d, nd, _ = po.build_copy_descs([(olay, blocks(load_ids))])
    po.execute(d, nd, host_is_src=True)
    assert np.array_equal(mem.read(dev), shadow)
    st = be.stats()
    assert st["device_status"] == 0
    if case["name"] in ("consecutive_ids_32k", "consecutive_ids_pitched") and route != "zerocopy":
        assert st["kernel_launches"] == 0 and st["dma_copies"] == 2 * n_ranges, "expected one DMA per range and direction"
    if case["name"] == "consecutive_ids_short_rows" and route != "zerocopy":
        assert st["kernel_launches"] > 0
    be.close()
    for a in allocs:
        pool.release(a[2])


def test_scattered_host_runs_and_many_layers(env):
    """Host images in many short runs (blocks saved at different times) across several layers:
    the zero-copy table path and the staged path are mixed inside one call."""
    pf, mem, pool, torch = env
    rng = np.random.default_rng(5)
    n_layers, num_blocks, seg = 5, 96, 16384
    be = pf.TransferBackend(0, min_dma_bytes=128 << 10, staging_slot_bytes=1 << 20)
    devs, inits, layers, images = [], [], [], []
    slab, slab_dev, handle = pool.alloc(n_layers * num_blocks * seg * 2)
    cursor = 0
    for li in range(n_layers):
        dev = mem.alloc(num_blocks * seg)
        init = rng.integers(0, 256, size=num_blocks * seg, dtype=np.uint8)
        mem.write(dev, init)
        ids = rng.permutation(num_blocks)[:64]
        runs, where = [], []
        first = 0
        for ln in (1, 20, 1, 1, 9, 32):   # run lengths: singles and longer runs
            cursor += seg * int(rng.integers(0, 3))   # gaps so runs never merge
            runs.append(pf.HostRun(first, ln, slab + cursor, slab_dev + cursor, seg))
            where.extend(cursor + i * seg for i in range(ln))
            cursor += ln * seg
            first += ln
        layers.append(pf.LayerXfer(dev.data_ptr(), seg, 0, seg, 1, list(ids), [runs]))
        devs.append(dev)
        inits.append(init)
        images.append((ids, where))
    events = [make_event(torch) for _ in range(n_layers)]
    be.save_layers(layers, 0, [e.cuda_event for e in events])
    hv = host_view(slab, n_layers * num_blocks * seg * 2)
    for li in (n_layers - 1, 0):
        events[li].synchronize()
    mem.sync()
    for li in range(n_layers):
        ids, where = images[li]
        for b, off in zip(ids, where):
            assert np.array_equal(hv[off:off + seg], inits[li][b * seg:(b + 1) * seg])
    for dev in devs:
        mem.zero(dev)
    be.load_layers(layers, 0, None)
    mem.sync()
    for li in range(n_layers):
        want = np.zeros(num_blocks * seg, dtype=np.uint8)
        for b in images[li][0]:
            want[b * seg:(b + 1) * seg] = inits[li][b * seg:(b + 1) * seg]
        assert np.array_equal(mem.read(devs[li]), want)
    st = be.stats()
    assert st["bytes_staged"] > 0 and st["bytes_zero_copy"] > 0 and st["device_status"] == 0
    be.close()
    pool.release(handle)


def test_empty_and_invalid_batches(env):
    pf, mem, pool, torch = env
    be = pf.TransferBackend(0)
    descs, n = be.make_descs([])
    be.d2h(descs, 0, 0)
    be.h2d(descs, 0, 0)
    be.save_layers([], 0, None)
    ev = make_event(torch)
    be.save_layers([pf.LayerXfer(0x1000, 16, 0, 16, 1, [], [[]])], 0, [ev.cuda_event])
    ev.synchronize()
    host, host_dev, handle = pool.alloc(4096)
    dev = mem.alloc(4096)
    with pytest.raises(pf.PegaflowInvalidArgument, match="host runs cover"):
        be.save_layers([pf.LayerXfer(dev.data_ptr(), 16, 0, 16, 1, [0, 1], [[pf.HostRun(0, 1, host, host_dev, 16)]])])
    with pytest.raises(pf.PegaflowInvalidArgument, match="n_ranges"):
        be.save_layers([pf.LayerXfer(dev.data_ptr(), 16, 0, 16, 3, [0], [[pf.HostRun(0, 1, host, host_dev, 16)]])])
    assert be.name() == "b200"
    be.close()
    pool.release(handle)


def test_pool_allocator_rules(env, kats):
    """allocator.rs:155-262 through the product pool: round-up, first offset, reuse after free."""
    pf, mem, pool, torch = env
    p = pf.PinnedPool(1 << 20, unit_hint=0)
    a = p.alloc(1)
    used, total, largest = p.usage()
    assert (used, total) == (512, 1 << 20) and largest == (1 << 20) - 512
    b = p.alloc(512)
    assert b[0] == a[0] + 512 and b[1] == a[1] + 512
    p.release(a[2])
    p.release(b[2])
    c = p.alloc(1024)
    assert c[0] == a[0]
    with pytest.raises(pf.PegaflowInternal, match="exhausted"):
        p.alloc(2 << 20)
    p.close()


def test_small_multi_layer_task_takes_one_launch(env):
    """A few blocks of many layers (the tail blocks saved while decoding) cost one kernel launch in
    each direction, and the per-layer events still fire."""
    pf, mem, pool, torch = env
    rng = np.random.default_rng(77)
    n_layers, num_blocks, seg = 12, 64, 8192
    be = pf.TransferBackend(0)
    devs, inits, layers = [], [], []
    ids = [5, 63, 1]
    slab, slab_dev, handle = pool.alloc(n_layers * 2 * len(ids) * seg)
    for li in range(n_layers):
        dev = mem.alloc(2 * num_blocks * seg)
        init = rng.integers(0, 256, size=2 * num_blocks * seg, dtype=np.uint8)
        mem.write(dev, init)
        off = li * 2 * len(ids) * seg
        runs = [[pf.HostRun(0, 3, slab + off + r * 3 * seg, slab_dev + off + r * 3 * seg, seg)] for r in range(2)]
        layers.append(pf.LayerXfer(dev.data_ptr(), seg, num_blocks * seg, seg, 2, ids, runs))
        devs.append(dev)
        inits.append(init)
    events = [make_event(torch) for _ in range(n_layers)]
    before = be.stats()["kernel_launches"]
    be.save_layers(layers, 0, [e.cuda_event for e in events])
    events[-1].synchronize()
    assert be.stats()["kernel_launches"] == before + 1
    hv = host_view(slab, n_layers * 2 * len(ids) * seg)
    for li in range(n_layers):
        for r in range(2):
            for i, b in enumerate(ids):
                o = li * 2 * 3 * seg + r * 3 * seg + i * seg
                src = r * num_blocks * seg + b * seg
                assert np.array_equal(hv[o:o + seg], inits[li][src:src + seg])
    for dev in devs:
        mem.zero(dev)
    be.load_layers(layers, 0, None)
    mem.sync()
    assert be.stats()["kernel_launches"] == before + 2
    for li in range(n_layers):
        want = np.zeros(2 * num_blocks * seg, dtype=np.uint8)
        for r in range(2):
            for b in ids:
                o = r * num_blocks * seg + b * seg
                want[o:o + seg] = inits[li][o:o + seg]
        assert np.array_equal(mem.read(devs[li]), want)
    assert be.stats()["device_status"] == 0
    be.close()
    pool.release(handle)


@pytest.mark.parametrize("route", ["staged", "zerocopy"])
def test_save_then_load_on_one_stream_needs_no_sync_in_between(env, route):
    """Stream order is the contract (transfer/mod.rs:15-16): a load enqueued right after a save on
    the same stream must see the bytes that save wrote, although the copies run on internal streams."""
    pf, mem, pool, torch = env
    rng = np.random.default_rng(99)
    num_blocks, seg, n = 1024, 65536, 384
    dev = mem.alloc(num_blocks * seg)
    host, host_dev, handle = pool.alloc(n * seg)
    be = pf.TransferBackend(0, route=ROUTES[route], staging_slot_bytes=4 << 20)
    stream = torch.cuda.Stream()
    src = rng.permutation(num_blocks // 2)[:n]
    dst = rng.permutation(num_blocks // 2)[:n] + num_blocks // 2
    runs = [[pf.HostRun(0, n, host, host_dev, seg)]]
    xs = pf.TransferBackend.make_layers([pf.LayerXfer(dev.data_ptr(), seg, 0, seg, 1, src, runs)])
    xl = pf.TransferBackend.make_layers([pf.LayerXfer(dev.data_ptr(), seg, 0, seg, 1, dst, runs)])
    for it in range(3):
        data = rng.integers(0, 256, size=num_blocks * seg, dtype=np.uint8)
        mem.write(dev, data)
        be.save_layers(xs, stream.cuda_stream)
        be.load_layers(xl, stream.cuda_stream)
        stream.synchronize()
        got = mem.read(dev).reshape(num_blocks, seg)
        assert np.array_equal(got[dst], data.reshape(num_blocks, seg)[src]), f"iteration {it}: stale host bytes loaded"
    be.close()
    pool.release(handle)


def test_gather_layers_runs_the_kernel_and_moves_nothing_to_the_host(env):
    """pf_backend_gather_layers (the timing aid behind bench.py's roofline figure): kernel launches,
    no DMA, the host image untouched; a real save on the same backend afterwards is still bit-exact;
    runs that would not be gathered are refused."""
    pf, mem, pool, torch = env
    rng = np.random.default_rng(21)
    num_blocks, seg, n = 200, 32768, 96
    region = 2 * num_blocks * seg
    dev = mem.alloc(region)
    init = rng.integers(0, 256, size=region, dtype=np.uint8)
    mem.write(dev, init)
    ids = rng.permutation(num_blocks)[:n]
    allocs = [pool.alloc(seg * n) for _ in range(2)]
    for a in allocs:
        host_view(a[0], seg * n)[:] = 0x5A
    runs = [[pf.HostRun(0, n, a[0], a[1], seg)] for a in allocs]
    be = pf.TransferBackend(0, min_dma_bytes=64 << 10, staging_slot_bytes=1 << 20)
    stream = torch.cuda.Stream()
    X = pf.LayerXfer(dev.data_ptr(), seg, num_blocks * seg, seg, 2, list(ids), runs)
    for _ in range(3):
        be.gather_layers([X], stream.cuda_stream)
    stream.synchronize()
    st = be.stats()
    assert st["kernel_launches"] >= 6 and st["dma_copies"] == 0 and st["bytes_zero_copy"] == 0
    assert st["device_status"] == 0
    for a in allocs:
        assert (host_view(a[0], seg * n) == 0x5A).all(), "gather_layers must not write host memory"
    assert np.array_equal(mem.read(dev), init), "gather_layers must not write the KV cache"
    # the same backend still saves correctly afterwards
    be.save_layers([X], stream.cuda_stream)
    stream.synchronize()
    for r, a in enumerate(allocs):
        got = host_view(a[0], seg * n).reshape(n, seg)
        want = init[r * num_blocks * seg:(r + 1) * num_blocks * seg].reshape(num_blocks, seg)[ids]
        assert np.array_equal(got, want)
    # refused: consecutive ids (a DMA, no kernel) and runs below the DMA threshold (zero-copy route)
    Xc = pf.LayerXfer(dev.data_ptr(), seg, num_blocks * seg, seg, 2, list(range(5, 5 + n)), runs)
    with pytest.raises(ValueError):
        be.gather_layers([Xc], stream.cuda_stream)
    short = [[pf.HostRun(0, 1, a[0], a[1], seg)] for a in allocs]
    Xs = pf.LayerXfer(dev.data_ptr(), seg, num_blocks * seg, seg, 2, [int(ids[0])], short)
    with pytest.raises(ValueError):
        be.gather_layers([Xs], stream.cuda_stream)
    be.close()
    for a in allocs:
        pool.release(a[2])


def test_staged_route_without_the_dependent_launch_attribute():
    """PEGAFLOW_B200_PDL=0 (read once per process) launches the gather/scatter kernel as a plain launch: the
    layer cases of the staged route, against the oracle, in a process that has the switch set."""
    import os
    import subprocess
    import sys

    proc = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu", os.path.abspath(__file__), "-k",
                           "test_layer_save_load_matches_oracle and staged"],
                          env=dict(os.environ, PEGAFLOW_B200_PDL="0"), cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                          stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert proc.returncode == 0 and " passed" in proc.stdout, proc.stdout[-2000:]
