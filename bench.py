#!/usr/bin/env python
"""Benchmark of the KV-cache save/load path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

A step is one pass of the hot path over one batch of synthetic input: the layer-wise save
(GPU -> pinned host pool) of every request of the workload followed by the warm load
(host pool -> GPU, into other block ids) of the same requests.  The workload is the
Llama-3.1-8B shape of the baseline (32 layers, 8 KV heads x 128, bf16, block 16; 8 requests of
10240 tokens = 640 blocks each at random block ids among 8192 GPU blocks; 10 GiB each way).
With N > 1 every rank runs that workload on its own GPU, stream and pool (weak scaling, no
data-path collective), in both arms; the b200 arm then adds a `peer` object: ranks N/2 .. N-1 act as
a second instance and pull prefix hits from ranks 0 .. N/2-1 over NVLink, across processes.

Prints ONE JSON line:  value = payload GB/s (10^9 B/s) with the KV cache resident in HBM,
timed with CUDA events; e2e = the same metric through the engine's public API (save with
hashes, prefix query, lease, load), host wall clock around a synchronised region.

Other modes (each prints one JSON line of its own):
    --workload W         the other baseline shapes (qwen3-0.6b, llama70b-tp8-rank, mla-bf16, mla-fp8, small) and
                         llama3.1-8b-crosslayer (the reference's default registration: one 2 MiB block per block id)
    --duplex             every step saves one set of blocks and loads another at the same time
    --peer [--peer-pairs K | --peer-local]
                         NVLink block copy between instances (GPU pairs, or both on one GPU)
    --transfer-grid      the reference's descriptor-level transfer_h2d grid on three backends
    --ttft               cold / warm time-to-first-token shape through the connector hooks
    --vllm-ttft [--after-forward]
                         the same shape under a real vLLM engine with this library as KV connector
    --pool-coldstart     pinned-pool allocation strategies
    --placement-probe    (with --gpus N) where in host memory a GPU's pool should lie: copy rates into chunks
                         allocated in different ways, one rank at a time and all ranks at once
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PCIE_GEN5_X16_GBS = 32e9 * 16 * (128 / 130) / 8 / 1e9   # 63.0 GB/s per direction before TLP overhead


def workloads():
    # name -> dict(layers, seg_bytes (K or V of one block), gpu_blocks, requests, blocks_per_request)
    # segments: 2 = K and V regions per layer (KV-first registration, one pool allocation per layer and
    # segment); 1 = one segment per block with page-first host pages (one page per block holding every layer).
    return {
        "llama3.1-8b": dict(layers=32, seg_bytes=16 * 8 * 128 * 2, gpu_blocks=8192, requests=8, blocks=640, segments=2),
        # the same model in the reference's default registration for non-MLA models: vLLM's cross-layer KV cache
        # [num_blocks, layers, 2, 16, 8, 128] registered as ONE pseudo-layer whose block is every layer's K and V,
        # 2 MiB (python/pegaflow/connector/__init__.py:67,170-171, worker.py:414-420); not page-first, direct backend
        "llama3.1-8b-crosslayer": dict(layers=1, seg_bytes=32 * 2 * 16 * 8 * 128 * 2, gpu_blocks=8192, requests=8,
                                       blocks=640, segments=1, page_first=False, mla=False),
        # Qwen3-0.6B round trip: 256 GPU blocks, 64 saved and loaded back into 64 other ids
        "qwen3-0.6b": dict(layers=28, seg_bytes=16 * 8 * 128 * 2, gpu_blocks=256, requests=1, blocks=64, segments=2),
        "small": dict(layers=4, seg_bytes=16 * 8 * 128 * 2, gpu_blocks=2048, requests=2, blocks=256, segments=2),
        # four layers of the llama3.1-8b shape with full-length requests: the same launches (20 MiB runs, three
        # to a gather launch) on 512 MiB of KV, small enough for a full ncu capture
        "llama3.1-8b-4layers": dict(layers=4, seg_bytes=16 * 8 * 128 * 2, gpu_blocks=2048, requests=2, blocks=640,
                                    segments=2),
        # one rank of Llama-3.1-70B TP=8: 1 KV head per rank -> 4 KiB segments, 4 prompts of 32768 tokens
        # (gpu_blocks leaves room for disjoint save and load ids when both directions run at once)
        "llama70b-tp8-rank": dict(layers=80, seg_bytes=16 * 1 * 128 * 2, gpu_blocks=16640, requests=4, blocks=2048,
                                  segments=2),
        # DeepSeek-V3-style latent cache [num_blocks, 64, 576], bf16 and fp8 byte widths
        "mla-bf16": dict(layers=61, seg_bytes=64 * 576 * 2, gpu_blocks=1024, requests=1, blocks=256, segments=1,
                         page_first=True, mla=True),
        "mla-fp8": dict(layers=61, seg_bytes=64 * 576 * 1, gpu_blocks=1024, requests=1, blocks=256, segments=1,
                        page_first=True, mla=True),
    }


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu_index), "-lms", "200"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_setup(n_gpus):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        import datetime

        # a rank that fails must not leave the others waiting for long
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=180))
    return rank, world, local


def barrier_and_max(value, world, device):
    """Barrier, then the max of `value` over ranks (device-side all-reduce)."""
    if world == 1:
        return value
    import torch
    import torch.distributed as dist

    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier(world):
    if world > 1:
        import torch.distributed as dist

        dist.barrier()


class Workload:
    """Synthetic KV cache in HBM + block id tables (seeded; stands in for a vLLM run)."""

    def __init__(self, spec, device, seed):
        import torch

        self.spec = spec
        self.device = device
        L, seg, nb = spec["layers"], spec["seg_bytes"], spec["gpu_blocks"]
        self.segments = spec["segments"]
        g = torch.Generator(device=device)
        g.manual_seed(seed)
        # per layer one tensor [2, num_blocks, seg] bytes (K region then V region, KV-first registration)
        # or [1, num_blocks, seg] for single-segment caches
        self.kv = []
        for _ in range(L):
            t = torch.empty((self.segments, nb, seg // 2), dtype=torch.bfloat16, device=device)
            t.normal_(0.0, 1.0, generator=g)
            self.kv.append(t.view(torch.uint8).view(self.segments, nb, seg))
        rng = np.random.default_rng(seed)
        n_req, per = spec["requests"], spec["blocks"]
        ids = rng.permutation(nb - 1)[: n_req * per] + 1          # id 0 is vLLM's null block
        self.save_ids = [ids[r * per:(r + 1) * per].astype(np.uint32) for r in range(n_req)]
        dst = rng.permutation(nb - 1)[: n_req * per] + 1
        self.load_ids = [dst[r * per:(r + 1) * per].astype(np.uint32) for r in range(n_req)]
        self.payload_per_request = L * per * self.segments * seg
        self.payload = self.payload_per_request * n_req

    def layer_ptr(self, layer):
        return self.kv[layer].data_ptr()

    @property
    def kv_stride(self):
        return self.spec["gpu_blocks"] * self.spec["seg_bytes"] if self.segments == 2 else 0

    @property
    def page_bytes(self):
        """Host page of one block when page-first: every layer's block back to back."""
        return self.spec["layers"] * self.spec["seg_bytes"]


def alloc_host_images(pool, wl):
    """Pool placement the engine would choose: split caches get one allocation per (request, layer,
    segment) with blocks back to back (offload.rs:477-508); single-segment caches get page-first pages,
    one per block, layer l at offset l * seg (offload.rs:182-282).  Returns per request, per layer, per
    range: (host, host_device, stride)."""
    L, seg, per = wl.spec["layers"], wl.spec["seg_bytes"], wl.spec["blocks"]
    out = []
    for _ in range(wl.spec["requests"]):
        if wl.segments == 2:
            req = []
            for _l in range(L):
                k, v = pool.alloc(per * seg), pool.alloc(per * seg)
                req.append([(k[0], k[1], seg), (v[0], v[1], seg)])
        else:
            pages = pool.alloc(per * wl.page_bytes)
            req = [[(pages[0] + l * seg, pages[1] + l * seg, wl.page_bytes)] for l in range(L)]
        out.append(req)
    return out


def make_layer_xfers(pf, wl, pool_allocs, ids_per_request):
    """One pre-marshalled LayerXfer array per request (32 layers, K and V runs)."""
    out = []
    seg = wl.spec["seg_bytes"]
    for r, ids in enumerate(ids_per_request):
        layers = []
        for l in range(wl.spec["layers"]):
            n = len(ids)
            runs = [[pf.HostRun(0, n, h, d, stride)] for (h, d, stride) in pool_allocs[r][l]]
            layers.append(pf.LayerXfer(wl.layer_ptr(l), seg, wl.kv_stride, seg, wl.segments, ids, runs))
        out.append(pf.TransferBackend.make_layers(layers))
    return out


def measure_pcie_ceiling(device, nbytes=1 << 30, iters=5, sustained=False, world=1):
    """One large pinned<->device cudaMemcpyAsync per direction (GB/s): best of `iters`, or with
    `sustained` the mean over `iters` back-to-back copies (for ranks that run it at the same time)."""
    import torch

    host = torch.empty(nbytes, dtype=torch.uint8, pin_memory=True)
    dev = torch.empty(nbytes, dtype=torch.uint8, device=device)
    res = {}
    for name, (dst, src) in {"d2h": (host, dev), "h2d": (dev, host)}.items():
        dst.copy_(src, non_blocking=True)
        torch.cuda.synchronize()
        if sustained:
            barrier(world)   # all ranks start a direction together
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(iters):
                dst.copy_(src, non_blocking=True)
            b.record()
            b.synchronize()
            res[name] = iters * nbytes / 1e6 / a.elapsed_time(b)
            continue
        best = 0.0
        for _ in range(iters):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            dst.copy_(src, non_blocking=True)
            b.record()
            b.synchronize()
            best = max(best, nbytes / 1e6 / a.elapsed_time(b))
        res[name] = best
    del host, dev
    return res


def duplex_pcie_ceiling(device, world, nbytes=1 << 30, iters=5):
    """Both directions at once: `iters` x 1 GiB pinned->device on one stream while as many go device->pinned on
    another, on every rank at the same time.  Per-rank GB/s of each direction (its own bytes over its own
    span) and of the pair (all bytes over the span from the first copy's start to the last one's end)."""
    import torch

    hosts = [torch.empty(nbytes, dtype=torch.uint8, pin_memory=True) for _ in range(2)]
    devs = [torch.empty(nbytes, dtype=torch.uint8, device=device) for _ in range(2)]
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    pairs = [(hosts[0], devs[0]), (devs[1], hosts[1])]       # (dst, src): d2h on stream 0, h2d on stream 1
    for (dst, src), s in zip(pairs, streams):
        with torch.cuda.stream(s):
            dst.copy_(src, non_blocking=True)
    torch.cuda.synchronize()
    barrier(world)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(2)]
    go = torch.cuda.Event()
    go.record()
    for (dst, src), s, (a, b) in zip(pairs, streams, ev):
        s.wait_event(go)
        with torch.cuda.stream(s):
            a.record()
            for _ in range(iters):
                dst.copy_(src, non_blocking=True)
            b.record()
    torch.cuda.synchronize()
    d2h = iters * nbytes / 1e6 / ev[0][0].elapsed_time(ev[0][1])
    h2d = iters * nbytes / 1e6 / ev[1][0].elapsed_time(ev[1][1])
    span = max(ev[0][0].elapsed_time(ev[0][1]), ev[0][0].elapsed_time(ev[1][1]), ev[1][0].elapsed_time(ev[0][1]),
               ev[1][0].elapsed_time(ev[1][1]))
    return {"d2h": d2h, "h2d": h2d, "pair": 2 * iters * nbytes / 1e6 / span}


def concurrent_pcie_ceiling(device, world):
    """What the host platform gives when every rank copies at once: per-rank sustained GB/s per
    direction, gathered on all ranks.  Several GPUs can share a root port, a socket link or the
    host's memory write bandwidth, so this, not `world` x the solo figure, bounds the N-GPU value."""
    import torch
    import torch.distributed as dist

    mine = measure_pcie_ceiling(device, sustained=True, world=world)
    t = torch.tensor([mine["d2h"], mine["h2d"]], dtype=torch.float64, device=device)
    every = [torch.zeros_like(t) for _ in range(world)]
    dist.all_gather(every, t)
    d2h = [round(float(x[0]), 2) for x in every]
    h2d = [round(float(x[1]), 2) for x in every]
    # the bench's value is bytes of all ranks over the slowest rank's time for a save pass plus a load pass
    slowest = max(1.0 / a + 1.0 / b for a, b in zip(d2h, h2d))
    return {"d2h_per_rank": d2h, "h2d_per_rank": h2d, "d2h_sum": round(sum(d2h), 2), "h2d_sum": round(sum(h2d), 2),
            "value_bound": round(2 * world / slowest, 2),
            "how": "every rank copies 5 x 1 GiB per direction at the same time; value_bound = 2 * ranks / "
                   "max over ranks of (1/d2h + 1/h2d), the same max-over-ranks rule as `value`"}


def cpu_baseline(wl, seconds_budget=8.0):
    """Host-core pool packing (oracle, kind "port"): memcpy gather of the same scattered blocks
    from a host shadow of two layers of the KV cache into the pool layout, 1 thread and all cores."""
    from oracle import pf_oracle as po
    from oracle import build_ref

    lib = C.CDLL(build_ref.build())
    lib.pfr_build.restype = C.c_void_p
    lib.pfr_build.argtypes = [C.c_void_p, C.c_size_t, C.POINTER(C.c_size_t), C.c_size_t, C.POINTER(C.c_size_t),
                              C.POINTER(C.c_double)]
    lib.pfr_free.argtypes = [C.c_void_p]
    spec = wl.spec
    seg, nb = spec["seg_bytes"], spec["gpu_blocks"]
    n_layers = min(2, spec["layers"])
    ids = np.concatenate(wl.save_ids).astype(np.uint64)
    # bounded sample: the host shadow of a layer is capped at 1 GiB, block ids wrap around inside it
    nb_full, nb = nb, max(1, min(nb, (1 << 30) // (spec["segments"] * seg)))
    if nb < nb_full:
        ids = ids[: min(len(ids), 1024)] % nb
    n = len(ids)
    rng = np.random.default_rng(1)
    nseg = spec["segments"]
    shadow = [rng.integers(0, 256, size=nseg * nb * seg, dtype=np.uint8) for _ in range(n_layers)]
    host = [np.zeros(nseg * n * seg, dtype=np.uint8) for _ in range(n_layers)]
    layers = (ref_layer_type() * n_layers)()
    for l in range(n_layers):
        lay = po.KVCacheLayout(shadow[l].ctypes.data, nseg * nb * seg, nb, seg, nb * seg if nseg == 2 else 0, nseg)
        layers[l].layout = lay.c
        for s in range(nseg):
            layers[l].host_base[s] = host[l].ctypes.data + s * n * seg
            layers[l].host_dev_base[s] = host[l].ctypes.data + s * n * seg
            layers[l].allocation[s] = 2 * l + s + 1
        layers[l].host_stride = seg
    nd, secs = C.c_size_t(), C.c_double()
    ids_c = (C.c_size_t * n)(*[int(x) for x in ids])
    descs = lib.pfr_build(layers, n_layers, ids_c, n, C.byref(nd), C.byref(secs))
    descs_p = C.cast(descs, C.POINTER(po.CopyDesc))
    payload = n_layers * n * nseg * seg
    cores = os.cpu_count() or 1
    out = {}
    for threads in (1, cores):
        po.execute(descs_p, nd.value, False, threads)   # warm
        t_total, passes = 0.0, 0
        while t_total < seconds_budget / 2 and passes < 64:
            t_total += po.execute(descs_p, nd.value, False, threads)
            passes += 1
        out[threads] = (payload * passes / t_total / 1e9, passes)
    # check the packed image once
    for l in range(n_layers):
        got = host[l][:seg]
        want = shadow[l][int(ids[0]) * seg:(int(ids[0]) + 1) * seg]
        assert np.array_equal(got, want)
    lib.pfr_free(descs)
    return {"value": round(out[cores][0], 2), "unit": "GB/s", "cores": cores, "kind": "port",
            "single_core_value": round(out[1][0], 2), "descriptor_build_seconds_per_M": round(secs.value / nd.value * 1e6, 3),
            "sample": f"{n_layers} of {spec['layers']} layers x {n} blocks"
                      + (" (all requests)" if nb == nb_full else f" (ids wrapped into a {nb}-block shadow)")
                      + f", {nseg} segment(s) per block, "
                      f"{payload / 2**20:.0f} MiB per pass, {out[cores][1]} passes, gather from a host shadow of the KV "
                      "cache into the pool layout with memcpy (save direction)"}


_REF_LAYER = None


def ref_layer_type():
    """ctypes mirror of `pfr_layer` (oracle/ref_path.cu); built on first use so that the product arm
    never touches the oracle package."""
    global _REF_LAYER
    if _REF_LAYER is None:
        from oracle.pf_oracle import Layout

        class RefLayer(C.Structure):
            _fields_ = [("layout", Layout), ("host_base", C.c_uint64 * 2), ("host_dev_base", C.c_uint64 * 2),
                        ("host_stride", C.c_size_t), ("allocation", C.c_size_t * 2)]

        _REF_LAYER = RefLayer
    return _REF_LAYER


class RefPinned:
    """Pinned, mapped host memory for the reference arm: one cudaHostAlloc(Mapped) region from
    oracle/ref_path.cu (pinned_mem.rs:153-163) handed out by a bump pointer in 512-byte units
    (the reference pool's default unit, pinned_pool.rs:135-141).  Nothing of the product is used."""

    def __init__(self, lib, nbytes):
        lib.pfr_host_alloc.argtypes = [C.c_size_t, C.POINTER(C.c_void_p), C.POINTER(C.c_uint64)]
        lib.pfr_host_free.argtypes = [C.c_void_p]
        host, dev = C.c_void_p(), C.c_uint64()
        rc = lib.pfr_host_alloc(nbytes, C.byref(host), C.byref(dev))
        if rc:
            raise RuntimeError(f"cudaHostAlloc of {nbytes} bytes failed with CUDA error {rc}")
        self.lib, self.host, self.dev, self.size, self.head = lib, host.value, dev.value, nbytes, 0

    def alloc(self, nbytes):
        off = self.head
        self.head += -(-nbytes // 512) * 512
        if self.head > self.size:
            raise RuntimeError("reference arm: pinned region exhausted")
        return self.host + off, self.dev + off, off

    def close(self):
        if self.host:
            self.lib.pfr_host_free(C.c_void_p(self.host))
            self.host = None


def run_reference(args, rank, world, local):
    """The reference's own transfer path restated (oracle/ref_path.cu): descriptor build on one host
    thread, its direct backend (one cudaMemcpyAsync per non-mergeable fragment), one sync per task.
    Every rank of a torchrun launch runs it on its own GPU, as every rank of the reference has its own
    GPU worker threads (gpu_worker.rs:131-201); the product library is not loaded."""
    import torch
    from oracle import build_ref
    from oracle import pf_oracle as po

    device = torch.device("cuda", local)
    spec = workloads()[args.workload]
    wl = Workload(spec, device, 42 + 2 + rank)
    lib = C.CDLL(build_ref.build())
    lib.pfr_build.restype = C.c_void_p
    lib.pfr_build.argtypes = [C.c_void_p, C.c_size_t, C.POINTER(C.c_size_t), C.c_size_t, C.POINTER(C.c_size_t),
                              C.POINTER(C.c_double)]
    lib.pfr_free.argtypes = [C.c_void_p]
    lib.pfr_submit_direct.argtypes = [C.c_void_p, C.c_size_t, C.c_int, C.c_void_p, C.POINTER(C.c_size_t)]
    lib.pfr_submit_kernel.argtypes = [C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]
    lib.pfr_sync.argtypes = [C.c_void_p]
    seg, L = spec["seg_bytes"], spec["layers"]
    per = spec["blocks"]
    pool = RefPinned(lib, wl.payload + (64 << 20))
    images = alloc_host_images(pool, wl)
    stream = torch.cuda.Stream()
    tasks = []
    for r in range(spec["requests"]):
        layers = (ref_layer_type() * L)()
        for l in range(L):
            lay = po.KVCacheLayout(wl.layer_ptr(l), wl.segments * spec["gpu_blocks"] * seg, spec["gpu_blocks"], seg,
                                   wl.kv_stride, wl.segments)
            layers[l].layout = lay.c
            for s, (h, d, stride) in enumerate(images[r][l]):
                layers[l].host_base[s], layers[l].host_dev_base[s] = h, d
                # page-first pages of one request come from one allocation; split layers from one each
                layers[l].allocation[s] = (r * L + l) * 2 + s + 1 if wl.segments == 2 else r + 1
                layers[l].host_stride = stride
        sids = (C.c_size_t * per)(*[int(x) for x in wl.save_ids[r]])
        lids = (C.c_size_t * per)(*[int(x) for x in wl.load_ids[r]])
        tasks.append((layers, sids, lids))
    stats = {"calls": 0, "build_s": 0.0}

    def task(layers, ids, host_is_src, kernel=False):
        nd, secs, calls = C.c_size_t(), C.c_double(), C.c_size_t()
        descs = lib.pfr_build(layers, L, ids, per, C.byref(nd), C.byref(secs))
        if kernel:
            rc = lib.pfr_submit_kernel(descs, nd.value, host_is_src, C.c_void_p(stream.cuda_stream))
        else:
            rc = lib.pfr_submit_direct(descs, nd.value, host_is_src, C.c_void_p(stream.cuda_stream), C.byref(calls))
        rc = rc or lib.pfr_sync(C.c_void_p(stream.cuda_stream))
        lib.pfr_free(descs)
        if rc:
            raise RuntimeError(f"reference path failed with CUDA error {rc}")
        stats["calls"] += calls.value
        stats["build_s"] += secs.value

    def step(kernel=False):
        t0 = time.perf_counter()
        for layers, sids, _ in tasks:
            task(layers, sids, 0, kernel)
        t1 = time.perf_counter()
        for layers, _, lids in tasks:
            task(layers, lids, 1, kernel)
        return t1 - t0, time.perf_counter() - t1

    # the reference picks its kernel backend for MLA models and the direct one otherwise
    # (python/pegaflow/connector/common.py:577-594)
    use_kernel = bool(spec.get("mla")) and bool(lib.pfr_has_reference_kernel())
    for _ in range(args.warmup):
        step(use_kernel)
    torch.cuda.synchronize()
    barrier(world)
    stats["calls"], stats["build_s"] = 0, 0.0
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    t_save = t_load = 0.0
    t0 = time.perf_counter()
    for _ in range(args.steps):
        a, b = step(use_kernel)
        t_save += a
        t_load += b
    torch.cuda.synchronize()
    elapsed = barrier_and_max(time.perf_counter() - t0, world, device)
    clocks = sampler.stop() if rank == 0 else None
    timed_calls, timed_build_s = stats["calls"], stats["build_s"]
    verified = verify_step(wl, lambda: step(use_kernel), torch, device)
    verified = barrier_and_max(0.0 if verified else 1.0, world, device) == 0.0
    extra = {}
    if lib.pfr_has_reference_kernel() and world == 1:
        ks, kl = step(kernel=not use_kernel)
        ks, kl = step(kernel=not use_kernel)
        other = {"save_gbs": round(wl.payload / ks / 1e9, 2), "load_gbs": round(wl.payload / kl / 1e9, 2)}
        if use_kernel:
            extra["reference_direct_backend"] = other
        else:
            other["note"] = ("the reference's own NVRTC kernel source compiled unchanged, 1 CTA x 256 threads per "
                             "fragment, pageable descriptor upload")
            extra["reference_kernel_backend"] = other
    pool.close()
    if rank != 0:
        return
    value = 2 * wl.payload * args.steps * world / elapsed / 1e9
    line = {
        "impl": "reference", "metric": "kv_save_load_GBps", "value": round(value, 3), "unit": "GB/s",
        "n_gpus": world, "ranks_measured": world, "bit_exact": bool(verified),
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(elapsed / args.steps * 1e3, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": {"workload": args.workload, **spec, "between_iterations": "inputs (10 GiB per direction) far exceed the 126 MB L2",
                   "path": ("reference kernel backend (its default for MLA): CPU descriptor build + pageable descriptor "
                            "upload + its own kernel + one sync per task (gpu_worker.rs:428-523, transfer/kernel.rs:79-135)")
                   if use_kernel else
                   ("reference direct backend restated: CPU descriptor build + merge + one cudaMemcpyAsync per "
                    "fragment + one sync per task (gpu_worker.rs:428-523, transfer/memcpy.rs:25-97)")},
        "save_gbs": round(wl.payload * args.steps / t_save / 1e9, 3), "load_gbs": round(wl.payload * args.steps / t_load / 1e9, 3),
        "frac_pcie_gen5_x16": round(value / world / PCIE_GEN5_X16_GBS, 4),
        "memcpy_calls_per_step": timed_calls // max(1, args.steps),
        "descriptor_build_ms_per_step": round(timed_build_s / max(1, args.steps) * 1e3, 2),
        "cpu_baseline": {"value": round(value, 3), "unit": "GB/s", "cores": world, "kind": "port",
                         "sample": "full workload on every rank; the reference drives its copy engines from one host "
                                   "thread per direction per GPU"},
        "e2e": {"value": round(value, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "clocks": clocks, **extra,
    }
    print(json.dumps(line))


def verify_step(wl, run_step, torch, device):
    """One more pass of the hot path, after the timed region, with every source block of every request
    and layer snapshotted first: afterwards every destination block must hold its source block's bits."""
    src = torch.from_numpy(np.concatenate(wl.save_ids).astype(np.int64)).to(device)
    dst = torch.from_numpy(np.concatenate(wl.load_ids).astype(np.int64)).to(device)
    snap = [kv[:, src].clone() for kv in wl.kv]
    torch.cuda.synchronize()
    run_step()
    torch.cuda.synchronize()
    ok = all(torch.equal(kv[:, dst], want) for kv, want in zip(wl.kv, snap))
    del snap
    return bool(ok)


def pool_images_match_gpu(wl, allocs, torch, device):
    """After a step's loads: for every request, layer and range, the destination blocks on the GPU equal
    the host images in the pool (read here through a CPU view of the pinned bytes, not by the library)."""
    seg, per = wl.spec["seg_bytes"], wl.spec["blocks"]
    for r, ids in enumerate(wl.load_ids):
        dst = torch.from_numpy(ids.astype(np.int64)).to(device)
        for l, ranges in enumerate(allocs[r]):
            for rng_i, (host, _dev, stride) in enumerate(ranges):
                span = (per - 1) * stride + seg
                view = np.ctypeslib.as_array((C.c_uint8 * span).from_address(host))
                rows = np.lib.stride_tricks.as_strided(view, shape=(per, seg), strides=(stride, 1))
                image = torch.from_numpy(np.ascontiguousarray(rows)).to(device)
                if not torch.equal(wl.kv[l][rng_i][dst], image):
                    return False
    return True


def spread(values):
    return {"min": round(min(values), 3), "median": round(statistics.median(values), 3), "max": round(max(values), 3)}


def time_gather_alone(args, pf, torch, local, route, wl, save_x, stream):
    """The gather kernel timed alone: the launches of one step's saves (same layers, same block
    ids, same grouping) enqueued back to back through pf_backend_gather_layers, which leaves the DMA
    out, between one CUDA event pair on the launching stream.  Returns None when the workload's runs
    do not take the staged route."""
    if route == 2 or args.contiguous_ids:
        return None
    be = pf.TransferBackend(local, route=route, time_kernels=False, staging_slot_bytes=args.slot_mib << 20,
                            staging_slots=args.slots, pack_ctas=args.pack_ctas, gather_slots=args.gather_slots)
    s = stream.cuda_stream
    try:
        for x in save_x:   # warm-up pass; also proves every run is a gathered one
            be.gather_layers(x, s)
    except ValueError:
        be.close()
        return None
    stream.synchronize()
    passes = int(min(64, max(3, -(-(8 << 30) // wl.payload))))
    n0 = be.stats()["kernel_launches"]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(passes):
        for x in save_x:
            be.gather_layers(x, s)
    e1.record(stream)
    stream.synchronize()
    ms = e0.elapsed_time(e1)
    st = be.stats()
    be.close()
    launches = st["kernel_launches"] - n0
    if launches <= 0 or ms <= 0 or st["dma_copies"] or st["device_status"]:
        return None
    return {"ms": ms, "launches": launches, "payload": wl.payload * passes, "passes": passes,
            "inputs_exceed_l2": wl.payload > 126e6}


# dram__bytes_read.sum + dram__bytes_write.sum (MB) of one 60 MiB save launch of copy_group_ldst under ncu
SAVE_LAUNCH_DRAM_MB = 62.929152 + 10.871808


def run_pair_overhead(args):
    """What a CUDA event pair around one gather or scatter launch measures beside the kernel: the same launches
    timed by event pairs and by the kernel's own clock, back to back (pf_backend_gather_layers) and inside the
    save and load pipelines, where every launch follows a wait for another stream's event."""
    import torch
    import pegaflow_b200 as pf

    device = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    wl = Workload(workloads()[args.workload], device, 42)
    pool = pf.PinnedPool(wl.payload + (64 << 20))
    allocs = alloc_host_images(pool, wl)
    stream = torch.cuda.Stream()
    s = stream.cuda_stream
    save_x = make_layer_xfers(pf, wl, allocs, wl.save_ids)
    load_x = make_layer_xfers(pf, wl, allocs, wl.load_ids)
    cases = [("gather launches back to back, no DMA", "gather_layers", save_x, {}),
             ("saves", "save_layers", save_x, {}), ("loads", "load_layers", load_x, {}),
             ("saves, one staging slot per launch", "save_layers", save_x, {"gather_slots": 1})]
    rows = []
    for name, method, xs, kw in cases:
        be = pf.TransferBackend(0, route=1, time_kernels=True, **kw)
        before = None
        for _ in range(3):              # one pass untimed, two counted
            for x in xs:
                getattr(be, method)(x, s)
            stream.synchronize()
            before = before or be.stats()
        after = be.stats()
        be.close()
        n = after["pack_kernel_launches"] - before["pack_kernel_launches"]
        dn = after["pack_kernel_device_launches"] - before["pack_kernel_device_launches"]
        pair_us = (after["pack_kernel_ms"] - before["pack_kernel_ms"]) / n * 1e3
        dev_us = (after["pack_kernel_device_ms"] - before["pack_kernel_device_ms"]) / max(1, dn) * 1e3
        rows.append({"case": name, "launches": n, "event_pair_us": round(pair_us, 2), "kernel_clock_us": round(dev_us, 2),
                     "pair_minus_kernel_us": round(pair_us - dev_us, 2),
                     "payload_mib_per_launch": round((after["pack_kernel_bytes"] - before["pack_kernel_bytes"]) / n / 2 / 2 ** 20, 1)})
    pool.close()
    print(json.dumps({"metric": "event_pair_overhead", "unit": "us", "workload": args.workload, "rows": rows,
                      "how": "per launch: one CUDA event pair on the launching stream (pf_backend_stats pack_kernel_ms) "
                             "against the kernel's own %globaltimer stamps, first CTA start to last CTA end "
                             "(pack_kernel_device_ms), over two passes of the workload's requests"}))


def build_roofline(stat_pairs, args, alone=None):
    """The `roofline` object.  `alone` (time_gather_alone) gives the headline figure: the kernel timed
    by itself with CUDA events.  The backend counters taken before and after the timed region (summed
    over `stat_pairs`, one pair per backend that ran in it) give the same kernel as it ran inside the
    save/load pipeline."""
    def delta(key):
        return sum(b[key] - a[key] for a, b in stat_pairs)

    pack_launches, pack_ms, pack_bytes = delta("pack_kernel_launches"), delta("pack_kernel_ms"), delta("pack_kernel_bytes")
    link_launches, link_ms, link_bytes = delta("link_kernel_launches"), delta("link_kernel_ms"), delta("link_kernel_bytes")
    dev_n, dev_ms = delta("pack_kernel_device_launches"), delta("pack_kernel_device_ms")
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    hbm_peak = peaks.get("hbm_gbs", 6650.0)
    if pack_launches and pack_ms > 0:
        ach = pack_bytes / 1e6 / pack_ms
        roofline = {"kernel": "copy_group_ldst (HBM gather/scatter of the staged route)", "bound": "hbm",
                    "achieved": round(ach, 1), "peak": hbm_peak, "unit": "GB/s", "frac": round(ach / hbm_peak, 4),
                    "peak_source": "measured (MEASURED_PEAKS.json)" if peaks else "fallback",
                    "launches": pack_launches, "avg_launch_us": round(pack_ms / pack_launches * 1e3, 2),
                    "algorithmic_bytes_per_launch": pack_bytes // pack_launches,
                    # DRAM bytes per launch: an ncu capture of a smaller case of the same kernel (8.398 MB read,
                    # 0 written per 8.389 MB of payload) scaled by payload
                    "traffic": args.traffic_per_launch if args.traffic_per_launch is not None
                    else round(pack_bytes / pack_launches / 2 * (8.398336 / 8.388608)),
                    "how": "one CUDA event pair around every launch, on the launching stream, inside the timed region"}
        if dev_n and dev_ms > 0:
            dev_ach = (pack_bytes / pack_launches) * dev_n / 1e6 / dev_ms
            roofline["note"] = ("an event pair around a ~8 us kernel also brackets its launch latency and the two event "
                                "records; `device_clock` is the same launches timed by the kernel's own clock: "
                                f"{round(dev_ach / hbm_peak, 4)} of peak")
            roofline["device_clock"] = {
                "avg_launch_us": round(dev_ms / dev_n * 1e3, 2), "achieved": round(dev_ach, 1),
                "frac": round(dev_ach / hbm_peak, 4), "launches": dev_n,
                "how": "the kernel's own %globaltimer stamps (first CTA start to last CTA end) for the same launches; "
                       "an event pair around a ~10 us kernel measures mostly the pair"}
        if alone:
            # headline: the kernel alone, back to back; what the pipeline run measured moves below it
            in_pipeline = {k: roofline.pop(k) for k in ("achieved", "frac", "launches", "avg_launch_us", "how")}
            for k in ("note", "device_clock"):
                if k in roofline:
                    in_pipeline[k] = roofline.pop(k)
            in_pipeline["how"] += (" (every launch there follows a wait for an event of the copy stream, and the copy "
                                   "engine bounds the step, so the stream is blocked when the launch comes up: a pair also "
                                   "brackets the 25-31 us the stream takes to resume after the wait, whatever the kernel's "
                                   "size, against 6 us of records and launch when launches are back to back; "
                                   "`bench.py --pair-overhead` measures both)")
            ach = 2 * alone["payload"] / 1e6 / alone["ms"]
            roofline.update({
                "achieved": round(ach, 1), "frac": round(ach / hbm_peak, 4), "launches": alone["launches"],
                "avg_launch_us": round(alone["ms"] / alone["launches"] * 1e3, 2),
                "algorithmic_bytes_per_launch": 2 * alone["payload"] // alone["launches"],
                "how": f"kernel timed alone: the gather launches of one step's saves (same layers, block ids and "
                       f"grouping), {alone['passes']} passes back to back without the DMA "
                       f"(pf_backend_gather_layers), one CUDA event pair on the launching stream around all of them; "
                       f"peak is the burst copy figure",
                "inputs_exceed_l2": alone["inputs_exceed_l2"],
                "in_pipeline": in_pipeline})
            if args.traffic_per_launch is None:
                # per launch of THIS leg, from an ncu capture of two 60 MiB save launches of the same kernel
                # (62.915 MB of payload each: 62.93 MB read; 9.49 and 12.25 MB written back while the launch ran,
                # the rest of the staging writes still being in L2 at its end), scaled by payload
                roofline["traffic"] = round(alone["payload"] / alone["launches"] * (SAVE_LAUNCH_DRAM_MB / 62.914560))
                roofline["traffic_how"] = ("dram__bytes_read.sum + dram__bytes_write.sum of a 60 MiB launch under ncu, "
                                           "scaled by payload: one read per payload byte, and the 0.15-0.19 of the "
                                           "staging writes that leave L2 before the launch ends")
    else:
        ach = link_bytes / 1e6 / link_ms if link_ms > 0 else 0.0
        roofline = {"kernel": "copy_units_tma (zero-copy over PCIe)", "bound": "hbm", "achieved": round(ach, 1),
                    "peak": hbm_peak, "unit": "GB/s", "frac": round(ach / hbm_peak, 4),
                    "note": "this kernel is bound by the PCIe link (128-byte TLPs: 53.1 of the 63.0 GB/s raw rate), not "
                            "HBM: see the `link` object",
                    "launches": link_launches, "traffic": args.traffic_per_launch}
    return roofline


def run_b200(args, rank, world, local):
    import torch
    import pegaflow_b200 as pf

    from pegaflow_b200 import sharding

    device = torch.device("cuda", local)
    spec = workloads()[args.workload]
    plan = sharding.rank_plan(rank, world, n_layers=spec["layers"], payload_bytes_per_rank=0, local_rank=local)
    wl = Workload(spec, device, plan.seed)
    L, seg, per, n_req = spec["layers"], spec["seg_bytes"], spec["blocks"], spec["requests"]
    if args.contiguous_ids:
        wl.save_ids = [np.arange(1 + r * per, 1 + (r + 1) * per, dtype=np.uint32) for r in range(n_req)]
        wl.load_ids = list(wl.save_ids)
    route = {"auto": 0, "staged": 1, "zerocopy": 2}[args.route]

    # ---------------- transfer-only arm: backend + pool, KV resident in HBM -------------------
    # each rank's pool on its GPU's own NUMA node (what the engine's per-node pools do)
    pool = pf.PinnedPool(wl.payload + (64 << 20), numa_node=pf.numa_node_of_device(local))
    allocs = alloc_host_images(pool, wl)
    be = pf.TransferBackend(local, route=route, time_kernels=not args.no_kernel_timing, link_ctas=args.link_ctas,
                            staging_slot_bytes=args.slot_mib << 20, staging_slots=args.slots,
                            copy_streams=args.copy_streams, pack_ctas=args.pack_ctas, gather_slots=args.gather_slots)
    save_x = make_layer_xfers(pf, wl, allocs, wl.save_ids)
    load_x = make_layer_xfers(pf, wl, allocs, wl.load_ids)
    stream = torch.cuda.Stream()
    s = stream.cuda_stream

    def step(events=None):
        if events:
            events[0].record(stream)
        for x in save_x:
            be.save_layers(x, s)
        if events:
            events[1].record(stream)
        for x in load_x:
            be.load_layers(x, s)
        if events:
            events[2].record(stream)

    for _ in range(max(3, args.warmup) if not args.allow_short_warmup else args.warmup):
        step()
    stream.synchronize()
    st0 = be.stats()
    barrier(world)
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    for k in range(args.steps):
        step(evs[k])
    stream.synchronize()
    torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    total_ms = evs[0][0].elapsed_time(evs[-1][2])
    save_ms = sum(e[0].elapsed_time(e[1]) for e in evs)
    load_ms = sum(e[1].elapsed_time(e[2]) for e in evs)
    total_ms = barrier_and_max(total_ms, world, device)
    st1 = be.stats()
    # Bit-exactness of the timed path, every request and layer.  (a) The last timed step's loads: each
    # destination block must hold what the pool held for it.  (b) One more step of the same calls with all
    # source blocks snapshotted first: every destination block must hold its source block's bits.
    verified = pool_images_match_gpu(wl, allocs, torch, device) and verify_step(wl, step, torch, device)
    verified = barrier_and_max(0.0 if verified else 1.0, world, device) == 0.0
    # per-layer events on one request (diagnostic, outside the timed region)
    lev = [torch.cuda.Event(enable_timing=True) for _ in range(L + 1)]
    for e in lev:
        e.record(stream)   # torch creates the cudaEvent_t on first record
    stream.synchronize()
    lev[0].record(stream)
    be.save_layers(save_x[0], s, [e.cuda_event for e in lev[1:]])
    stream.synchronize()
    torch.cuda.synchronize()
    layer_bytes = per * wl.segments * seg
    first_layer_ms = lev[0].elapsed_time(lev[1])
    all_layers_ms = max(lev[0].elapsed_time(lev[i + 1]) for i in range(L))
    st2 = be.stats()
    be.close()
    alone = time_gather_alone(args, pf, torch, local, route, wl, save_x, stream)
    del save_x, load_x
    pool.close()

    value = sharding.aggregate_throughput([2 * wl.payload * args.steps] * world, total_ms / 1e3)
    roofline = build_roofline([(st0, st1)], args, alone)

    # ---------------- end-to-end arm: the engine's public API ----------------------------------
    e2e, e2e_breakdown = None, None
    if not args.skip_e2e:
        e2e = run_e2e(args, pf, wl, rank, world, local, route)
        e2e_breakdown = e2e.pop("e2e_breakdown")

    concurrent = concurrent_pcie_ceiling(device, world) if world > 1 else None
    barrier(world)
    ceiling = measure_pcie_ceiling(device) if rank == 0 else None
    peer = peer_phase(args, pf, torch, rank, world, local) if world > 1 and not args.skip_peer else None
    cpu = None
    if rank == 0 and world == 1 and not args.skip_cpu_baseline:
        cpu = cpu_baseline(wl)
    if rank != 0:
        return
    save_gbs = wl.payload * args.steps / (save_ms / 1e3) / 1e9
    load_gbs = wl.payload * args.steps / (load_ms / 1e3) / 1e9
    line = {
        "metric": "kv_save_load_GBps", "value": round(value, 3), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(total_ms / args.steps, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": {"workload": args.workload, **spec, "route": args.route,
                   "between_iterations": "inputs (payload per direction per step far exceeds the 126 MB L2) are not "
                                         "re-read from cache; no flush needed",
                   "values": "bf16 N(0,1) from a seeded generator; block ids by seeded permutation without id 0"},
        "save_gbs": round(save_gbs, 3), "load_gbs": round(load_gbs, 3),
        "per_step": {"save_gbs": spread([wl.payload / 1e6 / e[0].elapsed_time(e[1]) for e in evs]),
                     "load_gbs": spread([wl.payload / 1e6 / e[1].elapsed_time(e[2]) for e in evs]),
                     "how": "rank 0, CUDA events around each timed step's saves and loads"},
        "bit_exact": bool(verified),
        "bit_exact_how": "every request and layer: the last timed step's destination blocks against the pool's host "
                         "images, then one more step with all source blocks snapshotted first",
        "link": {"bound": "pcie_gen5_x16", "peak_theoretical": round(PCIE_GEN5_X16_GBS, 2),
                 "save_frac": round(save_gbs / PCIE_GEN5_X16_GBS, 4), "load_frac": round(load_gbs / PCIE_GEN5_X16_GBS, 4),
                 "measured_ceiling_d2h": round(ceiling["d2h"], 2), "measured_ceiling_h2d": round(ceiling["h2d"], 2),
                 "save_frac_of_ceiling": round(save_gbs / ceiling["d2h"], 4),
                 "load_frac_of_ceiling": round(load_gbs / ceiling["h2d"], 4),
                 "ceiling_how": "one 1 GiB pinned<->device cudaMemcpyAsync per direction, best of 5, rank 0 alone",
                 "all_ranks_at_once": concurrent,
                 "value_frac_of_all_ranks_bound": round(value / concurrent["value_bound"], 4) if concurrent else None},
        "per_layer_save": {"first_layer_ms": round(first_layer_ms, 3), "all_layers_ms": round(all_layers_ms, 3),
                           "mean_layer_ms": round(all_layers_ms / L, 3), "layers": L,
                           "gbs": round(L * layer_bytes / 1e6 / all_layers_ms, 2),
                           "how": "per-layer completion events of one request: layer 0 is usable after "
                                  "first_layer_ms, the rest stream in behind it"},
        "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "e2e_breakdown": e2e_breakdown, "peer": peer,
        "gpu_launches": (st1["kernel_launches"] - st0["kernel_launches"]),
        "dma_copies": (st1["dma_copies"] - st0["dma_copies"]), "device_status": st2["device_status"],
        "clocks": clocks,
    }
    print(json.dumps(line))


def run_duplex(args, rank, world, local):
    """Save and load at the same time, as a serving rank does when one request's prefill is being
    offloaded while another's prefix is being fetched: the save backend and the load backend of one
    GPU run on their own streams, each driven by its own host thread (the engine's two workers per
    GPU, gpu_worker.rs:161-262).  PCIe is full duplex, so the two directions add up.

    Two sets of host images alternate: step k saves into set k % 2 while it loads from the other
    set, which the step before filled.  Block ids saved from and loaded into are disjoint."""
    import torch
    import pegaflow_b200 as pf

    device = torch.device("cuda", local)
    spec = workloads()[args.workload]
    wl = Workload(spec, device, 42 + 2 + rank)
    L, seg, per, n_req = spec["layers"], spec["seg_bytes"], spec["blocks"], spec["requests"]
    if 2 * n_req * per > spec["gpu_blocks"] - 1:
        raise SystemExit("--duplex needs gpu_blocks > 2 * requests * blocks")
    ids = np.random.default_rng(1000 + rank).permutation(spec["gpu_blocks"] - 1)[: 2 * n_req * per] + 1
    wl.save_ids = [ids[r * per:(r + 1) * per].astype(np.uint32) for r in range(n_req)]
    wl.load_ids = [ids[(n_req + r) * per:(n_req + r + 1) * per].astype(np.uint32) for r in range(n_req)]
    route = {"auto": 0, "staged": 1, "zerocopy": 2}[args.route]
    kw = dict(route=route, time_kernels=not args.no_kernel_timing, link_ctas=args.link_ctas,
              staging_slot_bytes=args.slot_mib << 20, staging_slots=args.slots, copy_streams=args.copy_streams,
              pack_ctas=args.pack_ctas)

    pool = pf.PinnedPool(2 * wl.payload + (64 << 20), numa_node=pf.numa_node_of_device(local))
    sets = [alloc_host_images(pool, wl) for _ in range(2)]
    be_save, be_load = pf.TransferBackend(local, **kw), pf.TransferBackend(local, **kw)
    save_x = [make_layer_xfers(pf, wl, a, wl.save_ids) for a in sets]
    load_x = [make_layer_xfers(pf, wl, a, wl.load_ids) for a in sets]
    s_save, s_load, main = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()

    from concurrent.futures import ThreadPoolExecutor

    threads = ThreadPoolExecutor(max_workers=2)

    def issue_saves(k):
        torch.cuda.set_device(local)
        for x in save_x[k % 2]:
            be_save.save_layers(x, s_save.cuda_stream)

    def issue_loads(k):
        torch.cuda.set_device(local)
        for x in load_x[(k + 1) % 2]:
            be_load.load_layers(x, s_load.cuda_stream)

    def step(k, events=None):
        # both directions start after everything of the step before (either stream) is done
        s_save.wait_stream(main)
        s_load.wait_stream(main)
        if events:
            events[0].record(s_save)
            events[1].record(s_load)
        jobs = [threads.submit(issue_saves, k), threads.submit(issue_loads, k)]
        for j in jobs:
            j.result()
        if events:
            events[2].record(s_save)
            events[3].record(s_load)
        main.wait_stream(s_save)
        main.wait_stream(s_load)
        if events:
            events[4].record(main)

    # prime set 1 so that step 0 has something to load; clear the destination blocks
    for x in save_x[1]:
        be_save.save_layers(x, s_save.cuda_stream)
    s_save.synchronize()
    every_dst = torch.from_numpy(np.concatenate(wl.load_ids).astype(np.int64)).to(device)
    every_src = torch.from_numpy(np.concatenate(wl.save_ids).astype(np.int64)).to(device)
    for l in range(L):
        wl.kv[l][:, every_dst] = 0
    torch.cuda.synchronize()

    warm = max(3, args.warmup) if not args.allow_short_warmup else args.warmup
    for k in range(warm):
        step(k)
    torch.cuda.synchronize()
    st0 = [be_save.stats(), be_load.stats()]
    barrier(world)
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(5)] for _ in range(args.steps)]
    first = torch.cuda.Event(enable_timing=True)
    first.record(main)
    for k in range(args.steps):
        step(warm + k, evs[k])
    torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    total_ms = barrier_and_max(first.elapsed_time(evs[-1][4]), world, device)
    save_ms = sum(e[0].elapsed_time(e[2]) for e in evs)
    load_ms = sum(e[1].elapsed_time(e[3]) for e in evs)
    st1 = [be_save.stats(), be_load.stats()]
    # bit-exactness of the timed path: what was loaded is what had been saved, for every layer
    verified = all(torch.equal(wl.kv[l][:, every_dst], wl.kv[l][:, every_src]) for l in range(L))
    status = be_save.stats()["device_status"] | be_load.stats()["device_status"]
    del save_x, load_x
    be_save.close()
    be_load.close()
    pool.close()
    threads.shutdown()

    value = 2 * wl.payload * args.steps * world / (total_ms / 1e3) / 1e9
    roofline = build_roofline(list(zip(st0, st1)), args)
    e2e = None
    if not args.skip_e2e:
        e2e = run_e2e(args, pf, wl, rank, world, local, route, duplex=True)
        e2e.pop("e2e_breakdown")
    concurrent = concurrent_pcie_ceiling(device, world) if world > 1 else None
    both = duplex_pcie_ceiling(device, world)
    if world > 1:
        import torch.distributed as dist

        t = torch.tensor([both["d2h"], both["h2d"], both["pair"]], dtype=torch.float64, device=device)
        every = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(every, t)
        both = {k: [round(float(x[i]), 2) for x in every] for i, k in enumerate(("d2h", "h2d", "pair"))}
    else:
        both = {k: [round(v, 2)] for k, v in both.items()}
    barrier(world)
    ceiling = measure_pcie_ceiling(device) if rank == 0 else None
    if rank != 0:
        return
    save_gbs = wl.payload * args.steps / (save_ms / 1e3) / 1e9
    load_gbs = wl.payload * args.steps / (load_ms / 1e3) / 1e9
    line = {
        "metric": "kv_save_load_GBps", "value": round(value, 3), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(total_ms / args.steps, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": {"workload": args.workload, **spec, "route": args.route,
                   "mode": "duplex: every step saves one set of blocks and loads another at the same time",
                   "between_iterations": "inputs (payload per direction per step far exceeds the 126 MB L2) are not "
                                         "re-read from cache; no flush needed",
                   "values": "bf16 N(0,1) from a seeded generator; disjoint save and load block ids by seeded permutation"},
        "save_gbs": round(save_gbs, 3), "load_gbs": round(load_gbs, 3), "bit_exact": bool(verified),
        "link": {"bound": "pcie_gen5_x16 full duplex", "peak_theoretical": round(2 * PCIE_GEN5_X16_GBS, 2),
                 "measured_ceiling_d2h": round(ceiling["d2h"], 2), "measured_ceiling_h2d": round(ceiling["h2d"], 2),
                 "value_frac_of_sum_of_ceilings": round(value / world / (ceiling["d2h"] + ceiling["h2d"]), 4),
                 "ceiling_how": "one 1 GiB pinned<->device cudaMemcpyAsync per direction, best of 5, one direction "
                                "at a time, rank 0 alone",
                 "all_ranks_at_once": concurrent,
                 "both_directions_at_once": {
                     "d2h_per_rank": both["d2h"], "h2d_per_rank": both["h2d"], "pair_per_rank": both["pair"],
                     "pair_sum": round(sum(both["pair"]), 2),
                     "value_frac": round(value / (world * min(both["pair"])), 4),
                     "how": "every rank runs 5 x 1 GiB plain cudaMemcpyAsync device->pinned on one stream and 5 x 1 GiB "
                            "pinned->device on another at the same time; value_frac = value / (ranks x the slowest "
                            "rank's pair rate), the max-over-ranks rule of `value`"}},
        "roofline": roofline, "cpu_baseline": None, "e2e": e2e,
        "gpu_launches": sum(b["kernel_launches"] - a["kernel_launches"] for a, b in zip(st0, st1)),
        "dma_copies": sum(b["dma_copies"] - a["dma_copies"] for a, b in zip(st0, st1)), "device_status": status,
        "clocks": clocks,
    }
    print(json.dumps(line))


def run_e2e(args, pf, wl, rank, world, local, route, duplex=False):
    """Same workload through the engine API: register, batch_save per request (hashes, dedupe, pinned
    allocation, GPU batch, cache insert), prefix query + lease, batch_load into other block ids."""
    import torch

    device = torch.device("cuda", local)
    spec = wl.spec
    L, seg, per, n_req = spec["layers"], spec["seg_bytes"], spec["blocks"], spec["requests"]
    steps_total = args.steps + max(1, args.warmup)
    # room for one and a half steps' blocks: older steps are evicted (LRU) while a new one is saved
    # (duplex: two steps' blocks are live at once, the one being saved and the one being loaded)
    eng = pf.PegaEngine((5 if duplex else 3) * wl.payload // 2 + (256 << 20), route=route, link_ctas=args.link_ctas,
                        staging_slot_bytes=args.slot_mib << 20, staging_slots=args.slots,
                        copy_streams=args.copy_streams)
    names = [f"model.layers.{l}.self_attn.attn" for l in range(L)]
    region = wl.segments * spec["gpu_blocks"] * seg
    eng.register_context_layer_batch_strided(
        "bench", "bench-ns", local, 0, 0, 1, 1, names, [wl.layer_ptr(l) for l in range(L)], [region] * L,
        [spec["gpu_blocks"]] * L, [seg] * L, [wl.kv_stride] * L, [wl.segments] * L, None, None,
        "kernel" if spec.get("mla") else "direct", bool(spec.get("page_first")))
    prepared = []
    for k in range(steps_total):
        reqs = []
        for r in range(n_req):
            hashes = [b"s%04dr%02d" % (k, r) + int(i).to_bytes(4, "little") for i in range(per)]
            saves = eng.prepare_saves([(names[l], wl.save_ids[r], hashes) for l in range(L)])
            reqs.append((saves, eng.prepare_hashes(hashes)))
        prepared.append(reqs)

    from concurrent.futures import ThreadPoolExecutor

    # Two caller threads, as a server handling concurrent save RPCs would have: while one request's
    # copy runs on the GPU worker, the next request's validation and pool allocation proceed.
    callers = ThreadPoolExecutor(max_workers=2)

    def step(k):
        if duplex:
            # this step's saves run while the blocks of the step before are loaded
            saving = [callers.submit(eng.batch_save, "bench", 0, 0, local, req[0]) for req in prepared[k]]
            load_from = k - 1
        else:
            if n_req == 1:      # one request: no second caller to overlap with
                eng.batch_save("bench", 0, 0, local, prepared[k][0][0])
            else:
                list(callers.map(lambda req: eng.batch_save("bench", 0, 0, local, req[0]), prepared[k]))
            eng.flush_saves()
            load_from = k
        pending = []
        for r, (_, hashes) in enumerate(prepared[load_from] if load_from >= 0 else []):
            blocks, missing = eng.query_prefix("bench", hashes)
            if missing:
                raise RuntimeError(f"prefix query missed {missing} blocks")
            lease = eng.create_query_lease("bench", blocks)
            pending.append(eng.batch_load_async("bench", 0, local, [names], [(lease, [wl.load_ids[r]])]))
        for p in pending:
            if p.wait(120) != 1:
                raise RuntimeError("load failed: " + p.error())
        if duplex:
            for f in saving:
                f.result()
            eng.flush_saves()

    for k in range(max(1, args.warmup)):
        step(k)
    torch.cuda.synchronize()
    barrier(world)
    ph0 = eng.phase_times()
    t0 = time.perf_counter()
    for k in range(args.steps):
        step(max(1, args.warmup) + k)
    torch.cuda.synchronize()
    mine = time.perf_counter() - t0
    elapsed = barrier_and_max(mine, world, device)
    ph1 = eng.phase_times()
    breakdown = {name: {"us_per_step": round((ph1[name][0] - ph0[name][0]) / args.steps * 1e6, 1),
                        "calls_per_step": round((ph1[name][1] - ph0[name][1]) / args.steps, 2)} for name in ph1}
    breakdown["step_us"] = round(mine / args.steps * 1e6, 1)
    breakdown["how"] = ("engine-side timers (pf_engine_get_phase_times), this rank, summed over the calls of a step; saves come "
                        "from two caller threads and loads are issued before any is awaited, so phases overlap and do not "
                        "add up to step_us; gpu.save_task / gpu.load_task are the workers' time from picking a task up to the "
                        "GPU being done, *.enqueue and *.queue_wait are parts of what their name prefixes")
    m = eng.metrics()
    callers.shutdown()
    eng.close()
    return {"value": round(2 * wl.payload * args.steps * world / elapsed / 1e9, 3), "unit": "GB/s",
            "h2d_bytes_per_step": wl.payload, "d2h_bytes_per_step": wl.payload,
            "ms_per_step": round(elapsed / args.steps * 1e3, 3), "clock": "host wall clock around a synchronised region",
            "api": "pf_engine_batch_save / flush_saves / query_prefix / create_query_lease / batch_load_inproc, "
                   "arguments marshalled once outside the timed region; saves issued from two caller threads (one request per "
                   "step: from the calling thread)"
                   + ("; each step's saves overlap the loads of the step before" if duplex else ""),
            "evicted_blocks": m["evicted_blocks"], "load_failures": m["load_failures"], "e2e_breakdown": breakdown}


def cuda_memcpy_async(dst_ptr, src_ptr, nbytes, stream):
    """cudaMemcpyAsync(cudaMemcpyDefault) on raw device addresses (torch cannot wrap a pointer that was
    opened from another process)."""
    rc = cudart().cudaMemcpyAsync(C.c_void_p(dst_ptr), C.c_void_p(src_ptr), nbytes, 4, C.c_void_p(stream))
    if rc:
        raise RuntimeError(f"cudaMemcpyAsync failed with CUDA error {rc}")


_CUDART = None


def cudart():
    """The CUDA runtime library torch has loaded, by ctypes."""
    import torch  # noqa: F401  (has loaded the CUDA runtime this resolves to)

    global _CUDART
    if _CUDART is None:
        for name in ("libcudart.so.12", "libcudart.so.13", "libcudart.so"):
            try:
                _CUDART = C.CDLL(name)
                break
            except OSError:
                continue
        else:
            raise RuntimeError("the CUDA runtime library is not loadable by name")
        _CUDART.cudaMemcpyAsync.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]
        _CUDART.cudaHostAlloc.argtypes = [C.POINTER(C.c_void_p), C.c_size_t, C.c_uint]
        _CUDART.cudaFreeHost.argtypes = [C.c_void_p]
    return _CUDART


class WriteCombinedChunk:
    """cudaHostAlloc(cudaHostAllocWriteCombined | cudaHostAllocPortable): host memory the CPU maps write-combining,
    which the device may then write without snooping the CPU's caches."""

    def __init__(self, nbytes):
        p = C.c_void_p()
        rc = cudart().cudaHostAlloc(C.byref(p), nbytes, 0x04 | 0x01)
        if rc:
            raise RuntimeError(f"cudaHostAlloc(WriteCombined) failed with CUDA error {rc}")
        self.addr = p.value

    def close(self):
        if self.addr:
            cudart().cudaFreeHost(C.c_void_p(self.addr))
            self.addr = None


def peer_phase(args, pf, torch, rank, world, local):
    """Same-box prefix sharing between two instances that live in different processes (the baseline's
    fifth configuration): ranks 0 .. N/2-1 are instance A, ranks N/2 .. N-1 instance B with the same TP degree.
    Every A rank owns a Qwen3-32B TP4-shard-shaped KV cache (64 layers, 2 KV heads per rank -> 8 KiB K and
    V segments, HND inside a block, 8192 blocks) and exports each layer's region (pf_ipc_export); the
    rank-aligned B rank opens them for its own GPU (pf_ipc_open_for) and pulls 4096 blocks (50 % of the prefix)
    of every layer into random block ids of its own cache with the peer-copy kernel - all pairs at the same
    time, no collective on the data path.  Compared with the same blocks going through a pinned host pool, and
    with one large device-to-device copy between the same two GPUs.  Returns the `peer` object on rank 0.

    Every rank takes part in every barrier whatever happens to it: a rank whose step fails (no peer access on
    this box, say) remembers why and skips its remaining work, and the object then says `unavailable`."""
    import torch.distributed as dist
    from pegaflow_b200 import _native as N
    from pegaflow_b200 import sharding

    half = world // 2
    device = torch.device("cuda", local)
    L, seg, nb, n = 64, 16 * 2 * 128 * 2, 8192, 4096
    who = sharding.peer_role(rank, world)
    role, pair = who.role, who.pair
    payload = L * n * 2 * seg
    gen = torch.Generator(device=device)
    st = {"error": None}      # this rank's state across the stages

    def stage(fn):
        if st["error"] is None:
            try:
                fn()
            except Exception as e:      # remembered; the barriers below still happen
                st["error"] = f"rank {rank}: {type(e).__name__}: {e}"[:300]

    def source_layers(seed):
        gen.manual_seed(seed)
        for _ in range(L):
            yield torch.randint(0, 256, (2, nb, seg), dtype=torch.uint8, device=device, generator=gen)

    rng = np.random.default_rng(4200 + pair)
    sids = (rng.permutation(nb - 1)[:n] + 1).astype(np.uint32)
    dids = (rng.permutation(nb - 1)[:n] + 1).astype(np.uint32)
    si = torch.from_numpy(sids.astype(np.int64)).to(device)
    di = torch.from_numpy(dids.astype(np.int64)).to(device)
    stream = torch.cuda.Stream()

    def exact():
        """Every layer: destination blocks hold the source blocks (regenerated here from A's seed), every
        other block is still zero."""
        ok = True
        for t, want_src in zip(st["dst"], source_layers(5000 + pair)):
            want = torch.zeros_like(t)
            want[:, di] = want_src[:, si]
            ok = ok and torch.equal(t, want)
            del want, want_src
        return ok

    # ---- A exports, B opens
    def a_export():
        st["kv"] = list(source_layers(5000 + pair))
        st["big"] = torch.empty(1 << 30, dtype=torch.uint8, device=device)
        regions = []
        for t in st["kv"] + [st["big"]]:
            r = N.IpcRegion()
            N.check(N.lib.pf_ipc_export(t.data_ptr(), t.numel(), C.byref(r)))
            regions.append(bytes(r))
        torch.cuda.synchronize()
        st["mine"] = regions

    if role == "A":
        stage(a_export)
    everyone = [None] * world
    dist.all_gather_object(everyone, st.get("mine"))

    def b_open_and_warm():
        if everyone[pair] is None:
            raise RuntimeError("the partner rank exported nothing")
        st["regions"] = [N.IpcRegion.from_buffer_copy(b) for b in everyone[pair]]
        st["src_ptrs"] = []
        for r in st["regions"]:     # mapped for this rank's GPU: its kernels and copies read A's memory over NVLink
            ptr, dev_id = C.c_uint64(), C.c_int()
            N.check(N.lib.pf_ipc_open_for(C.byref(r), local, C.byref(ptr), C.byref(dev_id)))
            st["src_ptrs"].append(ptr.value)
            st["src_dev"] = dev_id.value
        st["dst"] = [torch.zeros((2, nb, seg), dtype=torch.uint8, device=device) for _ in range(L)]
        st["be"] = pf.TransferBackend(local, link_ctas=args.link_ctas)
        st["sl"] = [(p_, seg, nb * seg, seg, 2, nb) for p_ in st["src_ptrs"][:L]]
        st["dl"] = [(t.data_ptr(), seg, nb * seg, seg, 2, nb) for t in st["dst"]]
        for _ in range(3):
            st["be"].peer_copy_layers(st["sl"], sids, st["dl"], dids, stream.cuda_stream)
        stream.synchronize()

    if role == "B":
        stage(b_open_and_warm)
    dist.barrier()          # all pairs start their timed copies together

    def b_timed():
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(args.steps):
            st["be"].peer_copy_layers(st["sl"], sids, st["dl"], dids, stream.cuda_stream)
        b.record(stream)
        b.synchronize()
        st["peer_ms"] = a.elapsed_time(b)

    if role == "B":
        stage(b_timed)
    dist.barrier()

    def b_check_and_ceiling():
        st["peer_exact"] = exact()
        st["stats"] = st["be"].stats()
        # ceiling: one 1 GiB device-to-device copy from the same peer GPU, best of 6, all pairs at once
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        scratch = torch.empty(1 << 30, dtype=torch.uint8, device=device)
        best = 0.0
        for _ in range(6):
            a.record(stream)
            cuda_memcpy_async(scratch.data_ptr(), st["src_ptrs"][L], 1 << 30, stream.cuda_stream)
            b.record(stream)
            b.synchronize()
            best = max(best, (1 << 30) / 1e6 / a.elapsed_time(b))
        st["ceiling"] = best
        st["be"].close()

    if role == "B":
        stage(b_check_and_ceiling)

    # ---- the reference's way: source GPU -> pinned host pool -> destination GPU.  Each half runs in the
    # process that owns the GPU (A saves its blocks into a pool, B loads as many bytes from a pool into its
    # blocks); a hit costs the sum of the two, since the load can only start when the save is in the pool.
    def half_setup():
        st["pool"] = pf.PinnedPool(payload + (64 << 20), numa_node=pf.numa_node_of_device(local))
        st["be_h"] = pf.TransferBackend(local)
        mem, ids = (st["kv"], sids) if role == "A" else (st["dst"], dids)
        lay, st["images"] = [], []
        for l in range(L):
            k, v = st["pool"].alloc(n * seg), st["pool"].alloc(n * seg)
            st["images"].append((k[0], v[0]))
            lay.append(pf.LayerXfer(mem[l].data_ptr(), seg, nb * seg, seg, 2, ids,
                                    [[pf.HostRun(0, n, k[0], k[1], seg)], [pf.HostRun(0, n, v[0], v[1], seg)]]))
        st["x"] = pf.TransferBackend.make_layers(lay)
        st["times"] = []

    def half_move():
        move = st["be_h"].save_layers if role == "A" else st["be_h"].load_layers
        torch.cuda.synchronize(device)
        t0 = time.perf_counter()
        move(st["x"], stream.cuda_stream)
        stream.synchronize()
        st["times"].append(time.perf_counter() - t0)

    def half_finish():
        st["half_s"], ok = min(st["times"]), True
        if role == "A":      # the pool now holds the source blocks of every layer
            for l in range(L):
                for r_i in range(2):
                    view = np.ctypeslib.as_array((C.c_uint8 * (n * seg)).from_address(st["images"][l][r_i])).reshape(n, seg)
                    ok = ok and torch.equal(st["kv"][l][r_i][si], torch.from_numpy(view).to(device))
        st["half_ok"] = ok and st["be_h"].stats()["device_status"] == 0
        st["be_h"].close(), st["pool"].close()

    if role:
        stage(half_setup)
    for _ in range(3):
        dist.barrier()
        if role:
            stage(half_move)
    if role:
        stage(half_finish)

    def b_close():
        for r in st["regions"]:
            N.check(N.lib.pf_ipc_close_for(C.byref(r), local))

    result = {"error": st["error"]}
    if role == "B":
        stage(b_close)
        if st["error"] is None:
            result = {"pair": [st["src_dev"], local], "ranks": [pair, rank],
                      "GBps": round(payload * args.steps / 1e6 / st["peer_ms"], 2), "ceiling_GBps": round(st["ceiling"], 1),
                      "bit_exact": bool(st["peer_exact"]), "ms": st["peer_ms"], "gpu_launches": st["stats"]["kernel_launches"],
                      "device_status": st["stats"]["device_status"], "load_half_s": st["half_s"],
                      "load_half_ok": bool(st["half_ok"]), "error": None}
        else:
            result = {"error": st["error"]}
    elif role == "A" and st["error"] is None:
        result = {"save_half_s": st["half_s"], "save_half_ok": bool(st["half_ok"]), "error": None}
    results = [None] * world
    dist.all_gather_object(results, result)
    dist.barrier()          # instance A keeps its memory until every B rank has closed its mappings
    st.clear()
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    errors = [r["error"] for r in results if r and r.get("error")]
    if errors:
        return {"unavailable": "; ".join(errors)}
    rs = [r for r in results if r and "pair" in r]
    for r in rs:    # a hit through the host pool: the A rank's save, then the B rank's load
        a_side = results[r["ranks"][0]]
        r["via_host_pool_GBps"] = round(payload / (a_side["save_half_s"] + r["load_half_s"]) / 1e9, 2)
        r["via_host_pool_ok"] = a_side["save_half_ok"] and r["load_half_ok"]
    agg = sum(payload * args.steps for _ in rs) / 1e6 / max(r["ms"] for r in rs)
    ceil_sum = sum(r["ceiling_GBps"] for r in rs)
    return {
        "config": {"workload": "qwen3-32b-tp4-rank prefix hit across instances", "layers": L, "seg_bytes": seg, "gpu_blocks": nb,
                   "blocks": n, "segments": 2, "payload_bytes_per_pair": payload,
                   "instances": "A = ranks 0..%d, B = ranks %d..%d, one process per GPU; B reaches A's KV cache through "
                                "pf_ipc_export / pf_ipc_open_for" % (half - 1, half, 2 * half - 1),
                   "kernel_runs_on": "destination GPU (pull)"},
        "pairs": [r["pair"] for r in rs], "per_pair_GBps": [r["GBps"] for r in rs], "aggregate_GBps": round(agg, 2),
        "link": {"bound": "nvlink5", "peak_nominal_per_direction": 900.0,
                 "measured_ceiling_per_pair": [r["ceiling_GBps"] for r in rs],
                 "frac_of_nominal": round(agg / (900.0 * len(rs)), 4), "frac_of_ceiling": round(agg / ceil_sum, 4),
                 "ceiling_how": "one 1 GiB device-to-device cudaMemcpyAsync from the same peer GPU, best of 6, every pair's "
                                "own measurement"},
        "via_host_pool_GBps": [r["via_host_pool_GBps"] for r in rs],
        "via_host_pool_how": "payload / (instance A's save of the hit blocks into a pinned pool + instance B's load of as many "
                             "bytes from a pinned pool), each half in the process that owns the GPU, all pairs at once, best of "
                             "3; A's pool images are compared with its cache for all layers: "
                             + ("equal" if all(r["via_host_pool_ok"] for r in rs) else "DIFFERENT"),
        "speedup_vs_host_pool": round(agg / max(1e-9, sum(r["via_host_pool_GBps"] for r in rs)), 2),
        "bit_exact": all(r["bit_exact"] for r in rs),
        "bit_exact_how": "all 64 layers of every pair, whole destination cache compared (copied blocks against the source "
                         "regenerated from its seed, all other blocks still zero) after the timed peer copies",
        "gpu_launches": sum(r["gpu_launches"] for r in rs), "device_status": max(r["device_status"] for r in rs),
        "how": "per pair: CUDA events on the destination rank's stream around `steps` calls of pf_backend_peer_copy_layers, "
               "all pairs released by one barrier; aggregate = all pairs' bytes / the slowest pair's time"}


def read_first_line(path):
    try:
        with open(path) as f:
            return f.readline().strip()
    except OSError:
        return None


def first_page_frame(addr):
    """Guest-physical page frame of the page at `addr` from /proc/self/pagemap (None when the kernel hides it)."""
    try:
        page = os.sysconf("SC_PAGESIZE")
        with open("/proc/self/pagemap", "rb") as f:
            f.seek(addr // page * 8)
            entry = int.from_bytes(f.read(8), "little")
        return (entry & ((1 << 55) - 1)) if entry >> 63 else None
    except OSError:
        return None


class WideChunk:
    """A 1 GiB anonymous mapping (2 MiB pages where the kernel grants them), touched, whose place in guest-physical
    memory is sampled at 16 points; pinned with cudaHostRegister only if it is kept."""

    def __init__(self, nbytes):
        import mmap

        self.nbytes = nbytes
        self.map = mmap.mmap(-1, nbytes, flags=mmap.MAP_PRIVATE | mmap.MAP_ANONYMOUS)
        if hasattr(mmap, "MADV_HUGEPAGE"):
            try:
                self.map.madvise(mmap.MADV_HUGEPAGE)
            except OSError:
                pass
        self.view = np.frombuffer(self.map, dtype=np.uint8)
        self.view[::4096] = 1
        self.addr = self.view.ctypes.data
        frames = [first_page_frame(self.addr + i * (nbytes // 16)) for i in range(16)]
        frames = sorted(f for f in frames if f is not None)
        self.frames_gib = [round(f * 4096 / 2 ** 30, 1) for f in frames]
        self.median_gib = self.frames_gib[len(frames) // 2] if frames else -1.0
        self.registered = False

    def register(self, torch):
        rc = torch.cuda.cudart().cudaHostRegister(self.addr, self.nbytes, 0)
        if int(rc) != 0:
            raise RuntimeError(f"cudaHostRegister failed with {int(rc)}")
        self.registered = True

    def close(self, torch=None):
        if self.registered:
            import torch as _torch

            _torch.cuda.cudart().cudaHostUnregister(self.addr)
            self.registered = False
        self.view = None
        self.map.close()


def run_placement_probe(args, rank, world, local):
    """Does it matter where in host memory a GPU's pinned pool lies?  On a guest that shows a single NUMA
    node the kernel gives no answer, so this measures it: every rank allocates candidate chunks in several
    ways (cudaHostAlloc or mmap + pre-touch + cudaHostRegister; from threads restricted to each quarter of the
    CPUs; early and late in the process's life), then times plain cudaMemcpyAsync copies between its GPU and
    each chunk - one rank at a time, and with all ranks copying at once - and finally all ranks at once into
    each rank's best chunk.  Prints one JSON line with the whole table."""
    import torch
    import torch.distributed as dist
    import pegaflow_b200 as pf

    device = torch.device("cuda", local)
    chunk = args.probe_chunk_mib << 20
    piece = min(chunk, 256 << 20)
    cpus = sorted(os.sched_getaffinity(0))
    quarters = [cpus[i * len(cpus) // 4:(i + 1) * len(cpus) // 4] or cpus for i in range(4)]
    kinds = [("cudaHostAlloc", q, {}) for q in range(4)] + [("mmap+register", q, {"use_mmap": True}) for q in range(4)] \
        + [("mmap+madvise(HUGEPAGE)+register", None, {"transparent_huge": True})] \
        + [("cudaHostAlloc-late", None, {}) for _ in range(args.probe_late_chunks)]
    if args.probe_hugepages:
        kinds.append(("hugepages", None, {"use_hugepages": True}))
    chunks = []
    for name, q, kw in kinds:
        os.sched_setaffinity(0, quarters[q] if q is not None else cpus)
        try:
            pool = pf.PinnedPool(chunk + (1 << 20), **kw)
            host, host_dev, _ = pool.alloc(chunk)
            chunks.append({"kind": name, "cpu_quarter": q, "pool": pool, "host": host, "pfn": first_page_frame(host)})
        except pf.PegaFlowError as e:
            chunks.append({"kind": name, "cpu_quarter": q, "pool": None, "unavailable": str(e)[:100]})
    os.sched_setaffinity(0, cpus)
    try:
        w = WriteCombinedChunk(chunk)
        chunks.append({"kind": "cudaHostAlloc(WriteCombined)", "cpu_quarter": None, "pool": w, "host": w.addr,
                       "pfn": first_page_frame(w.addr)})
    except RuntimeError as e:
        chunks.append({"kind": "cudaHostAlloc(WriteCombined)", "cpu_quarter": None, "pool": None, "unavailable": str(e)[:100]})
    # a sweep over guest-physical memory: every rank fills `probe_wide_gib` GiB at the same time (together
    # they reach far into the guest's memory), keeps the chunks that lie lowest, highest and in between, and
    # gives the rest back before anything is pinned
    wide = []
    if args.probe_wide_gib > 0:
        wide = [WideChunk(chunk) for _ in range(args.probe_wide_gib * (1 << 30) // chunk)]
        barrier(world)
        wide.sort(key=lambda w: w.median_gib)
        picks = sorted({round(i * (len(wide) - 1) / 3) for i in range(4)})
        for i, w in enumerate(wide):
            if i not in picks:
                w.close()
        wide = [wide[i] for i in picks]
        for w in wide:
            w.register(torch)
            chunks.append({"kind": "mmap(2 MiB pages)+register, sweep", "cpu_quarter": None, "pool": w, "host": w.addr,
                           "pfn": first_page_frame(w.addr), "frames_gib_min_median_max":
                               [w.frames_gib[0], w.median_gib, w.frames_gib[-1]] if w.frames_gib else None})
    dev = torch.empty(piece, dtype=torch.uint8, device=device)
    stream = torch.cuda.Stream()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def copy_rate(c, to_host, reps, piece=piece):
        """GB/s of `reps` passes over the chunk in pieces of 256 MiB (or of `piece` bytes)."""
        a.record(stream)
        for _ in range(reps):
            for off in range(0, chunk, piece):
                if to_host:
                    cuda_memcpy_async(c["host"] + off, dev.data_ptr(), piece, stream.cuda_stream)
                else:
                    cuda_memcpy_async(dev.data_ptr(), c["host"] + off, piece, stream.cuda_stream)
        b.record(stream)
        b.synchronize()
        return reps * chunk / 1e6 / a.elapsed_time(b)

    live = [c for c in chunks if c["pool"] is not None]
    for c in live:                       # first use of every chunk, untimed
        copy_rate(c, True, 1), copy_rate(c, False, 1)
    for turn in range(world):            # one rank at a time
        barrier(world)
        if turn == rank:
            for c in live:
                c["solo_d2h"], c["solo_h2d"] = round(copy_rate(c, True, 1), 2), round(copy_rate(c, False, 1), 2)
    for i, c in enumerate(chunks):       # every rank at once, chunk i of each
        for key, to_host in (("all_d2h", True), ("all_h2d", False)):
            barrier(world)
            if c["pool"] is not None:
                c[key] = round(copy_rate(c, to_host, args.probe_reps), 2)
    best = {k: max(live, key=lambda c: c[k]) for k in ("all_d2h", "all_h2d")}
    final = {}
    for key, to_host in (("all_d2h", True), ("all_h2d", False)):     # every rank at once, each into its best chunk
        barrier(world)
        final[key] = round(copy_rate(best[key], to_host, args.probe_reps), 2)
        barrier(world)
        final[key + "_first_chunk"] = round(copy_rate(live[0], to_host, args.probe_reps), 2)
    # how the rate of one GPU falls as more GPUs copy at once: ranks 0..k-1 copy, the others wait
    ladder = {}
    counts = sorted({k for k in (1, 2, 3, 4, 6, 8, world) if k <= world})
    for key, to_host in (("d2h", True), ("h2d", False)):
        for k in counts:
            barrier(world)
            ladder[f"{key}_{k}_at_once"] = round(copy_rate(live[0], to_host, args.probe_reps), 2) if rank < k else None
            barrier(world)
    # even ranks write host memory while odd ranks read it, then the other way round
    mixed = {}
    for name, flip in (("even_d2h_odd_h2d", 0), ("even_h2d_odd_d2h", 1)):
        barrier(world)
        to_host = (rank + flip) % 2 == 0
        mixed[name] = {"dir": "d2h" if to_host else "h2d", "gbs": round(copy_rate(live[0], to_host, args.probe_reps), 2)}
    # the sizes the engine's own copies have: one staging slot, and one block-sized item
    by_piece = {}
    for mib in (32, 2):
        for key, to_host in (("d2h", True), ("h2d", False)):
            barrier(world)
            by_piece[f"all_{key}_{mib}mib_pieces"] = round(copy_rate(live[0], to_host, 1, mib << 20), 2)
    mine = {"rank": rank, "gpu": local,
            "chunks": [{k: v for k, v in c.items() if k not in ("pool", "host")} for c in chunks],
            "best_chunk": {k: chunks.index(v) for k, v in best.items()}, "all_ranks_best_chunk": final,
            "ranks_at_once": ladder, "mixed_directions": mixed, "piece_size": by_piece}
    for c in live:
        c["pool"].close()
    every = [None] * world
    if world > 1:
        dist.all_gather_object(every, mine)
    else:
        every = [mine]
    if rank != 0:
        return

    def total(key):
        return round(sum(r["all_ranks_best_chunk"][key] for r in every), 2)

    print(json.dumps({
        "metric": "pinned_pool_placement_probe", "unit": "GB/s", "n_gpus": world, "host_cpus": len(cpus),
        "numa_nodes_visible": pf._native.lib.pf_numa_num_nodes(), "chunk_mib": args.probe_chunk_mib,
        "transparent_hugepage": read_first_line("/sys/kernel/mm/transparent_hugepage/enabled"),
        "nr_hugepages": read_first_line("/proc/sys/vm/nr_hugepages"),
        "how": "plain cudaMemcpyAsync in 256 MiB pieces between each rank's GPU and each of its candidate chunks; solo_* = "
               "one rank at a time, all_* = every rank at once on its chunk of the same index; all_ranks_best_chunk = every "
               "rank at once, each on the chunk that was fastest for it under load (and on its first chunk, for comparison)",
        "ranks_at_once_sum": {k: round(sum(r["ranks_at_once"][k] or 0.0 for r in every), 2) for k in every[0]["ranks_at_once"]},
        "piece_size_sum": {k: round(sum(r["piece_size"][k] for r in every), 2) for k in every[0]["piece_size"]},
        "mixed_directions_sum": {name: {d: round(sum(r["mixed_directions"][name]["gbs"] for r in every
                                                     if r["mixed_directions"][name]["dir"] == d), 2) for d in ("d2h", "h2d")}
                                 for name in every[0]["mixed_directions"]},
        "sum_all_ranks_best_chunk": {"d2h": total("all_d2h"), "h2d": total("all_h2d"),
                                     "d2h_first_chunk": total("all_d2h_first_chunk"),
                                     "h2d_first_chunk": total("all_h2d_first_chunk")},
        "ranks": every}))



def peer_pairs_phase(pf, torch, n_pairs, args, L, seg, nb, n):
    """`n_pairs` prefix hits at once: instance B's rank i (GPU n_pairs + i) pulls the blocks of instance A's
    rank i (GPU i), rank-aligned shards of two instances with the same TP degree.  No collective."""
    payload = L * n * 2 * seg
    pairs = []
    for i in range(n_pairs):
        s_dev, d_dev = i, n_pairs + i
        rng = np.random.default_rng(4200 + i)
        ds, dd = torch.device("cuda", s_dev), torch.device("cuda", d_dev)
        src = [torch.randint(0, 256, (2, nb, seg), dtype=torch.uint8, device=ds) for _ in range(L)]
        dst = [torch.zeros((2, nb, seg), dtype=torch.uint8, device=dd) for _ in range(L)]
        sids = (rng.permutation(nb - 1)[:n] + 1).astype(np.uint32)
        dids = (rng.permutation(nb - 1)[:n] + 1).astype(np.uint32)
        pf.enable_peer_access(d_dev, s_dev)
        be = pf.TransferBackend(d_dev, link_ctas=args.link_ctas)
        torch.cuda.set_device(d_dev)
        pairs.append(dict(src=src, dst=dst, sids=sids, dids=dids, be=be, stream=torch.cuda.Stream(device=dd),
                          sl=[(t.data_ptr(), seg, nb * seg, seg, 2) for t in src],
                          dl=[(t.data_ptr(), seg, nb * seg, seg, 2) for t in dst], dev=d_dev, ds=ds, dd=dd))

    def enqueue(steps, events=False):
        for p in pairs:
            torch.cuda.set_device(p["dev"])
            if events:
                p["a"] = torch.cuda.Event(enable_timing=True)
                p["b"] = torch.cuda.Event(enable_timing=True)
                p["a"].record(p["stream"])
            for _ in range(steps):
                p["be"].peer_copy_layers(p["sl"], p["sids"], p["dl"], p["dids"], p["stream"].cuda_stream)
            if events:
                p["b"].record(p["stream"])

    def sync_all():
        for p in pairs:
            p["stream"].synchronize()

    enqueue(max(3, args.warmup))
    sync_all()
    ok = True
    for p in pairs:
        si = torch.from_numpy(p["sids"].astype(np.int64))
        di = torch.from_numpy(p["dids"].astype(np.int64))
        ok = ok and all(torch.equal(p["dst"][l][:, di.to(p["dd"])].cpu(), p["src"][l][:, si.to(p["ds"])].cpu())
                        for l in (0, L - 1))
    t0 = time.perf_counter()
    enqueue(args.steps, events=True)
    sync_all()
    wall = time.perf_counter() - t0
    per_pair = [round(payload * args.steps / 1e6 / p["a"].elapsed_time(p["b"]), 2) for p in pairs]
    status = 0
    for p in pairs:
        status |= p["be"].stats()["device_status"]
        p["be"].close()
    return {"pairs": [[i, n_pairs + i] for i in range(n_pairs)], "per_pair_GBps": per_pair,
            "aggregate_GBps": round(n_pairs * payload * args.steps / wall / 1e9, 2), "bit_exact": bool(ok),
            "device_status": status,
            "how": "per pair: CUDA events on the pair's stream; aggregate: all pairs' bytes over the host wall clock "
                   "from the first enqueue to the last stream's completion"}


def run_peer_local(args):
    """The peer-copy kernel with source and destination on one GPU (two instances sharing a device, or a
    profiling run on a single-GPU box): every byte is read from and written to HBM, so the kernel is timed
    against the HBM roofline instead of NVLink."""
    import torch
    import pegaflow_b200 as pf

    L, seg, nb, n = args.peer_layers, 16 * 2 * 128 * 2, 8192, 4096
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    rng = np.random.default_rng(42 + 5)
    src = [torch.randint(0, 256, (2, nb, seg), dtype=torch.uint8, device=dev) for _ in range(L)]
    dst = [torch.zeros((2, nb, seg), dtype=torch.uint8, device=dev) for _ in range(L)]
    sids = (rng.permutation(nb - 1)[:n] + 1).astype(np.uint32)
    dids = (rng.permutation(nb - 1)[:n] + 1).astype(np.uint32)
    payload = L * n * 2 * seg
    be = pf.TransferBackend(0, link_ctas=args.link_ctas)
    stream = torch.cuda.Stream()
    sl = [(t.data_ptr(), seg, nb * seg, seg, 2) for t in src]
    dl = [(t.data_ptr(), seg, nb * seg, seg, 2) for t in dst]
    for _ in range(max(1, args.warmup)):
        be.peer_copy_layers(sl, sids, dl, dids, stream.cuda_stream)
    stream.synchronize()
    si, di = torch.from_numpy(sids.astype(np.int64)).to(dev), torch.from_numpy(dids.astype(np.int64)).to(dev)
    ok = all(torch.equal(dst[l][:, di], src[l][:, si]) for l in (0, L - 1))
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(stream)
    for _ in range(args.steps):
        be.peer_copy_layers(sl, sids, dl, dids, stream.cuda_stream)
    b.record(stream)
    b.synchronize()
    ms = a.elapsed_time(b) / args.steps
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    hbm = peaks.get("hbm_gbs", 6650.0)
    st = be.stats()
    print(json.dumps({
        "metric": "kv_peer_copy_local_GBps", "value": round(payload / 1e6 / ms, 1), "unit": "GB/s", "n_gpus": 1,
        "steps": args.steps, "higher_is_better": True, "dtype": "u8", "data": "synthetic", "bit_exact": bool(ok),
        "config": {"workload": "qwen3-32b-tp4-rank prefix hit, both instances on one GPU", "layers": L, "seg_bytes": seg,
                   "blocks": n},
        "roofline": {"kernel": "copy_peer_warp", "bound": "hbm", "achieved": round(2 * payload / 1e6 / ms, 1), "peak": hbm,
                     "unit": "GB/s", "frac": round(2 * payload / 1e6 / ms / hbm, 4),
                     "algorithmic_bytes_per_step": 2 * payload, "launches_per_step": st["kernel_launches"] // (args.steps + max(1, args.warmup)),
                     "how": "one CUDA event pair around all launches of the timed steps"},
        "gpu_launches": st["kernel_launches"], "device_status": st["device_status"]}))


def run_peer(args):
    """Same-box prefix hit: blocks of instance A (GPU 0) land in other block ids of instance B (GPU 1),
    over NVLink with the peer-copy kernel and, for comparison, through the pinned host pool.
    Qwen3-32B TP4 shard shape: 64 layers, 2 KV heads per rank -> 8 KiB segments, 4096 of 8192 blocks."""
    import torch
    import pegaflow_b200 as pf

    if args.peer_local:
        return run_peer_local(args)
    if torch.cuda.device_count() < 2:
        print(json.dumps({"metric": "kv_peer_copy_GBps", "unavailable": "needs two GPUs on one box"}))
        return
    L, seg, nb, n = 64, 16 * 2 * 128 * 2, 8192, 4096
    d0, d1 = torch.device("cuda", 0), torch.device("cuda", 1)
    rng = np.random.default_rng(42 + 5)
    src = [torch.randint(0, 256, (2, nb, seg), dtype=torch.uint8, device=d0) for _ in range(L)]
    dst = [torch.zeros((2, nb, seg), dtype=torch.uint8, device=d1) for _ in range(L)]
    sids = (rng.permutation(nb - 1)[:n] + 1).astype(np.uint32)
    dids = (rng.permutation(nb - 1)[:n] + 1).astype(np.uint32)
    payload = L * n * 2 * seg
    # The kernel runs on the destination GPU and reads across NVLink (pull), or with --peer-push on the
    # source GPU and writes across it (push).
    run_on = 0 if args.peer_push else 1
    pf.enable_peer_access(run_on, 1 - run_on)
    be = pf.TransferBackend(run_on, link_ctas=args.link_ctas)
    torch.cuda.set_device(run_on)
    stream = torch.cuda.Stream(device=torch.device("cuda", run_on))

    src_layouts = [(src[l].data_ptr(), seg, nb * seg, seg, 2) for l in range(L)]
    dst_layouts = [(dst[l].data_ptr(), seg, nb * seg, seg, 2) for l in range(L)]

    def peer_step():
        # what the engine's peer_load does: every layer of the hit in one call
        be.peer_copy_layers(src_layouts, sids, dst_layouts, dids, stream.cuda_stream)

    for _ in range(max(3, args.warmup)):
        peer_step()
    stream.synchronize()
    si, di = torch.from_numpy(sids.astype(np.int64)), torch.from_numpy(dids.astype(np.int64))
    ok = all(torch.equal(dst[l][:, di.to(d1)].cpu(), src[l][:, si.to(d0)].cpu()) for l in (0, L - 1))
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(stream)
    for _ in range(args.steps):
        peer_step()
    b.record(stream)
    b.synchronize()
    peer_gbs = payload * args.steps / 1e6 / a.elapsed_time(b)
    # ceiling: one large device-to-device copy across NVLink
    big0 = torch.empty(1 << 30, dtype=torch.uint8, device=d0)
    big1 = torch.empty(1 << 30, dtype=torch.uint8, device=d1)
    best = 0.0
    for _ in range(6):
        a.record(stream)
        with torch.cuda.stream(stream):
            big1.copy_(big0, non_blocking=True)
        b.record(stream)
        b.synchronize()
        best = max(best, (1 << 30) / 1e6 / a.elapsed_time(b))
    del big0, big1
    # the reference's way today: GPU 0 -> pinned host pool -> GPU 1
    pool = pf.PinnedPool(payload + (64 << 20))
    be0, be1 = pf.TransferBackend(0), pf.TransferBackend(1)
    st0, st1 = torch.cuda.Stream(device=d0), torch.cuda.Stream(device=d1)
    layers_save, layers_load = [], []
    for l in range(L):
        k, v = pool.alloc(n * seg), pool.alloc(n * seg)
        runs = [[pf.HostRun(0, n, k[0], k[1], seg)], [pf.HostRun(0, n, v[0], v[1], seg)]]
        layers_save.append(pf.LayerXfer(src[l].data_ptr(), seg, nb * seg, seg, 2, sids, runs))
        layers_load.append(pf.LayerXfer(dst[l].data_ptr(), seg, nb * seg, seg, 2, dids, runs))
    xs, xl = pf.TransferBackend.make_layers(layers_save), pf.TransferBackend.make_layers(layers_load)
    t_host = []
    for _ in range(3):
        torch.cuda.synchronize(d0)
        torch.cuda.synchronize(d1)
        t0 = time.perf_counter()
        be0.save_layers(xs, st0.cuda_stream)
        st0.synchronize()
        be1.load_layers(xl, st1.cuda_stream)
        st1.synchronize()
        t_host.append(time.perf_counter() - t0)
    host_gbs = payload / min(t_host) / 1e9
    stats = be.stats()
    concurrent = None
    if args.peer_pairs > 1:
        if torch.cuda.device_count() < 2 * args.peer_pairs:
            concurrent = {"unavailable": f"{args.peer_pairs} pairs need {2 * args.peer_pairs} GPUs"}
        else:
            del src, dst
            be.close(), be0.close(), be1.close(), pool.close()
            torch.cuda.empty_cache()
            concurrent = peer_pairs_phase(pf, torch, args.peer_pairs, args, L, seg, nb, n)
    print(json.dumps({
        "metric": "kv_peer_copy_GBps", "value": round(peer_gbs, 2), "unit": "GB/s", "n_gpus": 2, "steps": args.steps,
        "higher_is_better": True, "dtype": "u8", "data": "synthetic", "bit_exact": bool(ok),
        "config": {"workload": "qwen3-32b-tp4-rank prefix hit", "kernel_runs_on": "source GPU (push)" if args.peer_push
                   else "destination GPU (pull)", "layers": L, "seg_bytes": seg, "gpu_blocks": nb,
                   "blocks": n, "segments": 2},
        "link": {"bound": "nvlink5", "peak_nominal": 900.0, "measured_ceiling": round(best, 1),
                 "frac_of_nominal": round(peer_gbs / 900.0, 4), "frac_of_ceiling": round(peer_gbs / best, 4),
                 "ceiling_how": "one 1 GiB device-to-device copy GPU0 -> GPU1, best of 6"},
        "via_host_pool_GBps": round(host_gbs, 2), "speedup_vs_host_pool": round(peer_gbs / host_gbs, 2),
        "concurrent_pairs": concurrent,
        "gpu_launches": stats["kernel_launches"], "device_status": stats["device_status"]}))


def run_ttft(args):
    """The reference's KV-cache benchmark shape (README.md:89-94: Llama-3.1-8B, 8 prompts of 10 K tokens,
    1-token decode) replayed on one GPU through the worker-connector hooks, with synthetic layers standing
    in for the model (torch matmuls and attention of the model's sizes, random weights shared by all layers).

    cold = prefill of the whole prompt + save of its KV blocks; warm = prefix load + one decode token.
    "after_forward" follows the reference's worker: nothing moves until the whole forward pass is over — its
    save_kv_layer is empty and wait_for_save hands all layers to a save thread that first synchronises the
    device (worker.py:755-800, 884-888); its wait_for_layer_load is empty too, so a load must be complete
    before the request is scheduled (worker.py:549-713).  "layerwise" uses the per-layer hooks this library
    fills in: every layer's save is queued behind an event recorded after that layer's compute, and the
    decode step waits per layer on the layer's load event.  For a cold request both the time to the first
    token and the time until the KV blocks are in the pool (when the request's blocks may be reused) are
    reported; the save is never on the first token's path, it only finishes earlier."""
    import torch
    import torch.nn.functional as F
    import pegaflow_b200 as pf
    from pegaflow_b200 import connector

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    L, H, NQ, NKV, D, FFN, BS = 32, 4096, 32, 8, 128, 14336, 16
    T, n_req, nb = 10240, args.ttft_requests, 8192
    per = T // BS
    g = torch.Generator(device=dev)
    g.manual_seed(7)

    def rnd(*shape, scale=0.02):
        return (torch.randn(*shape, generator=g, device=dev, dtype=torch.float32) * scale).to(torch.bfloat16)

    w_qkv, w_o, w_gu, w_d = rnd(H, (NQ + 2 * NKV) * D), rnd(NQ * D, H), rnd(H, 2 * FFN), rnd(FFN, H)
    names = [f"model.layers.{l}.self_attn.attn" for l in range(L)]
    caches = {n: torch.zeros((2, nb, BS, NKV, D), dtype=torch.bfloat16, device=dev) for n in names}
    eng = pf.PegaEngine((2 * n_req + 2) * (L * per * 2 * BS * NKV * D * 2) + (256 << 20))
    conn = connector.PegaWorkerConnector(connector.InProcEngineClient(eng), eng, instance_id="ttft", namespace="ttft-ns",
                                         device_id=0, block_size=BS)
    conn.register_kv_caches(caches)
    rng = np.random.default_rng(11)
    compute = torch.cuda.Stream()

    def layer_prefill(x, cache, ids):
        x = F.rms_norm(x, (H,))
        qkv = x @ w_qkv
        q, k, v = qkv.split([NQ * D, NKV * D, NKV * D], dim=-1)
        cache[0][ids] = k.view(per, BS, NKV, D)          # the layer's attention writes its KV pages
        cache[1][ids] = v.view(per, BS, NKV, D)
        a = F.scaled_dot_product_attention(q.view(1, T, NQ, D).transpose(1, 2), k.view(1, T, NKV, D).transpose(1, 2),
                                           v.view(1, T, NKV, D).transpose(1, 2), is_causal=True, enable_gqa=True)
        x = x + a.transpose(1, 2).reshape(T, NQ * D) @ w_o
        gate, up = (x @ w_gu).chunk(2, dim=-1)
        return x + (F.silu(gate) * up) @ w_d

    def layer_decode(x, cache, ids):
        x = F.rms_norm(x, (H,))
        qkv = x @ w_qkv
        q, _k, _v = qkv.split([NQ * D, NKV * D, NKV * D], dim=-1)
        k = cache[0][ids].view(1, T, NKV, D).transpose(1, 2)   # reads the pages the load brought in
        v = cache[1][ids].view(1, T, NKV, D).transpose(1, 2)
        a = F.scaled_dot_product_attention(q.view(1, 1, NQ, D).transpose(1, 2), k, v, enable_gqa=True)
        x = x + a.transpose(1, 2).reshape(1, NQ * D) @ w_o
        gate, up = (x @ w_gu).chunk(2, dim=-1)
        return x + (F.silu(gate) * up) @ w_d

    def cold(mode, r):
        ids_np = (rng.permutation(nb - 1)[:per] + 1)
        ids = torch.from_numpy(ids_np.astype(np.int64)).to(dev)
        hashes = [b"%s-c%02d-" % (mode.encode(), r) + int(i).to_bytes(4, "little") for i in range(per)]
        ids_list = ids_np.tolist()
        x = rnd(T, H, scale=1.0)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        events = []
        with torch.cuda.stream(compute):
            for name in names:
                x = layer_prefill(x, caches[name], ids)
                if mode == "layerwise":
                    ev = torch.cuda.Event()
                    ev.record(compute)
                    events.append(ev)        # must outlive the save that waits on it
                    conn.save_kv_layer(name, ids_list, hashes, ev.cuda_event)
        compute.synchronize()
        first_token_ms = (time.perf_counter() - t0) * 1e3
        if mode == "after_forward":
            torch.cuda.synchronize()
            conn.wait_for_save([(name, ids_list, hashes) for name in names])
        else:
            conn.wait_for_save()
        return first_token_ms, (time.perf_counter() - t0) * 1e3, hashes, ids_np

    def warm(mode, r, hashes):
        dst_np = (rng.permutation(nb - 1)[:per] + 1)
        dst = torch.from_numpy(dst_np.astype(np.int64)).to(dev)
        for c in caches.values():
            c[:, dst] = 0
        x = rnd(1, H, scale=1.0)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        q = conn.client.query_prefetch("ttft", hashes, f"{mode}-w{r}")
        if q.num_hit_blocks != per:
            raise RuntimeError(f"prefix query hit {q.num_hit_blocks} of {per} blocks")
        conn.start_load_kv([(f"{mode}-w{r}", q.lease, dst_np.tolist())])
        if mode == "after_forward":
            done = []
            while not done:
                done, failed = conn.get_finished()
                if failed:
                    raise RuntimeError("load failed")
        with torch.cuda.stream(compute):
            for name in names:
                if mode == "layerwise":
                    conn.wait_for_layer_load(name, compute.cuda_stream)
                x = layer_decode(x, caches[name], dst)
        compute.synchronize()
        ms = (time.perf_counter() - t0) * 1e3
        if mode == "layerwise":
            done = []
            while not done:
                done, failed = conn.get_finished()
                if failed:
                    raise RuntimeError("load failed")
        return ms, x.float().cpu()

    # warm-up of kernels, allocator and pool (not reported)
    _, _, h0, _ = cold("after_forward", 99)
    warm("after_forward", 99, h0)
    modes = ("after_forward", "layerwise")
    first_token = {m_: [] for m_ in modes}
    saved_at = {m_: [] for m_ in modes}
    warm_ms = {m_: [] for m_ in modes}
    saved, same = {}, True
    for r in range(n_req):
        for mode in modes:
            ft, sv, hashes, _ = cold(mode, r)
            first_token[mode].append(ft)
            saved_at[mode].append(sv)
            saved[(mode, r)] = hashes
    for r in range(n_req):
        # both warm modes load the same stored prompt into the same destination blocks and feed the same
        # token: the outputs must be identical bit for bit, or a layer was consumed before it had landed
        outs = {}
        state, gstate = rng.bit_generator.state, g.get_state()
        for mode in modes:
            rng.bit_generator.state = state
            g.set_state(gstate)
            ms, out = warm(mode, r, saved[("layerwise", r)])
            warm_ms[mode].append(ms)
            outs[mode] = out
        # bit patterns, not values: equal NaNs must count as equal
        same = same and torch.equal(outs["after_forward"].view(torch.int32), outs["layerwise"].view(torch.int32)) \
            and bool(torch.isfinite(outs["after_forward"]).all())
    m = eng.metrics()
    conn.unregister()
    eng.close()

    def summary(v):
        return {"mean_ms": round(float(np.mean(v)), 2), "max_ms": round(float(np.max(v)), 2)}

    kv_gib = L * per * 2 * BS * NKV * D * 2 / 2**30
    print(json.dumps({
        "metric": "ttft_shape_ms", "unit": "ms", "higher_is_better": False, "n_gpus": 1, "data": "synthetic",
        "config": {"workload": "llama3.1-8b, prompts of 10240 tokens, 1-token decode", "requests": n_req,
                   "kv_gib_per_request": round(kv_gib, 3), "layers": L,
                   "model": "synthetic layers of the model's sizes (torch matmul + SDPA, random weights)"},
        "cold_first_token": {k: summary(v) for k, v in first_token.items()},
        "cold_kv_in_pool": {k: summary(v) for k, v in saved_at.items()},
        "warm_first_token": {k: summary(v) for k, v in warm_ms.items()},
        "cold_kv_in_pool_earlier_by_ms": round(float(np.mean(saved_at["after_forward"]) - np.mean(saved_at["layerwise"])), 2),
        "warm_first_token_earlier_by_ms": round(float(np.mean(warm_ms["after_forward"]) - np.mean(warm_ms["layerwise"])), 2),
        "warm_outputs_identical": bool(same), "load_failures": m["load_failures"],
        "published_reference": {"cold_mean_ms": 572.5, "warm_mean_ms": 61.5,
                                "note": "README.md:89-94: H800, real vLLM serving at 4 req/s; context only"}}))


def run_vllm_ttft(args):
    """The reference's KV-cache benchmark (README.md:89-94: Llama-3.1-8B, 8 prompts of 10 K tokens, 1-token
    decode) under a real vLLM engine with this library as its KV connector.  The model has the published
    architecture sizes and random weights (there are no checkpoints here); prompts are random token ids.
    cold = first time a prompt is seen (prefill + save), warm = the same prompt after vLLM's own prefix cache
    was reset, so its KV comes from the host pool.  One process per hook mode (--after-forward selects the
    reference's behaviour)."""
    os.environ.setdefault("VLLM_ENABLE_V1_MULTIPROCESSING", "0")
    os.environ.setdefault("VLLM_LOGGING_LEVEL", "WARNING")
    import tempfile

    from transformers import LlamaConfig
    from vllm import LLM, SamplingParams
    from vllm.config import KVTransferConfig

    from pegaflow_b200 import vllm_connector

    layerwise = not args.after_forward
    model_dir = tempfile.mkdtemp(prefix="llama31-8b-shape-")
    LlamaConfig(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32,
                num_key_value_heads=8, head_dim=128, max_position_embeddings=131072, rope_theta=500000.0,
                torch_dtype="bfloat16", architectures=["LlamaForCausalLM"]).save_pretrained(model_dir)
    n_req, prompt_len = args.ttft_requests, 10240
    llm = LLM(model=model_dir, load_format="dummy", skip_tokenizer_init=True, enforce_eager=True, max_model_len=12288,
              max_num_batched_tokens=16384, gpu_memory_utilization=0.5, dtype="bfloat16", seed=0,
              enable_prefix_caching=True, block_size=16,
              kv_transfer_config=KVTransferConfig(
                  kv_connector="PegaKVConnector", kv_connector_module_path="pegaflow_b200.vllm_connector", kv_role="kv_both",
                  kv_connector_extra_config={"pegaflow.pool_bytes": (n_req + 3) * (5 << 28),
                                             "pegaflow.layerwise": layerwise}))
    rng = np.random.default_rng(17)
    prompts = [{"prompt_token_ids": rng.integers(1, 120000, size=prompt_len).tolist()} for _ in range(n_req)]
    one = SamplingParams(temperature=0.0, max_tokens=1, detokenize=False)
    engine = next(iter(vllm_connector._ENGINES.values()))

    def timed(p):
        t0 = time.perf_counter()
        out = llm.generate([p], one, use_tqdm=False)
        return (time.perf_counter() - t0) * 1e3, out[0].outputs[0].token_ids[0]

    warmup = {"prompt_token_ids": rng.integers(1, 120000, size=prompt_len).tolist()}
    timed(warmup)
    timed(warmup)
    cold = [timed(p) for p in prompts]
    saved = engine.metrics()["save_bytes"]
    timed({"prompt_token_ids": [5, 6, 7]})             # one more step: finished requests' blocks are released
    reset_ok = llm.reset_prefix_cache()
    loaded0 = engine.metrics()["load_bytes"]
    warm = [timed(p) for p in prompts]
    m = engine.metrics()

    def summary(v):
        ms = [x for x, _ in v]
        return {"mean_ms": round(float(np.mean(ms)), 2), "max_ms": round(float(np.max(ms)), 2)}

    print(json.dumps({
        "metric": "vllm_ttft_ms", "unit": "ms", "higher_is_better": False, "n_gpus": 1, "data": "synthetic",
        "config": {"workload": "vLLM, Llama-3.1-8B sizes with random weights, prompts of 10240 random tokens, 1-token decode, "
                               "one request at a time, eager mode", "requests": n_req,
                   "hooks": "layerwise" if layerwise else "after_forward"},
        "cold": summary(cold), "warm_from_host_pool": summary(warm),
        "warm_speedup": round(float(np.mean([x for x, _ in cold]) / np.mean([x for x, _ in warm])), 2),
        "same_first_token": [t for _, t in cold] == [t for _, t in warm], "prefix_cache_reset": bool(reset_ok),
        "saved_gib": round(saved / 2**30, 3), "loaded_gib": round((m["load_bytes"] - loaded0) / 2**30, 3),
        "load_failures": m["load_failures"],
        "published_reference": {"cold_mean_ms": 572.5, "warm_mean_ms": 61.5,
                                "note": "README.md:89-94: H800, real checkpoint, serving at 4 req/s; context only"}}))
    sys.stdout.flush()
    vllm_connector.close_shared_engines()
    os._exit(0)


def run_transfer_grid(args):
    """The reference's descriptor-level micro-benchmark (pegaflow-core/benches/transfer_h2d.rs:23-33, 301-339)
    on three backends: 4096-byte fragments x {1 Ki, 4 Ki, 16 Ki, 64 Ki} x {contiguous, every other device
    block, shuffled descriptor order} x {D2H, H2D}, 3 warm-up + 20 timed submissions, each followed by a stream
    synchronise, host clock.  Backends: this library through `pf_backend_d2h/h2d` on the same `CopyDesc` array
    (the narrowest drop-in), the reference's direct backend and its kernel backend (oracle/ref_path.cu)."""
    import torch
    import pegaflow_b200 as pf
    from pegaflow_b200 import _native as N
    from oracle import build_ref

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    seg, counts, warm, iters = 4096, [1024, 4096, 16384, 65536], 3, 20
    ref = C.CDLL(build_ref.build())
    ref.pfr_submit_direct.argtypes = [C.c_void_p, C.c_size_t, C.c_int, C.c_void_p, C.POINTER(C.c_size_t)]
    ref.pfr_submit_kernel.argtypes = [C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]
    ref.pfr_sync.argtypes = [C.c_void_p]
    has_kernel = bool(ref.pfr_has_reference_kernel())
    pool = pf.PinnedPool(max(counts) * seg + (1 << 20))
    host, host_dev, _ = pool.alloc(max(counts) * seg)
    device = torch.empty(((max(counts) - 1) * 2 + 1) * seg, dtype=torch.uint8, device=dev)
    hview = np.ctypeslib.as_array(C.cast(host, C.POINTER(C.c_uint8)), shape=(max(counts) * seg,))
    hview[:] = (np.arange(hview.size, dtype=np.uint64) * 31 + 7).astype(np.uint8)
    be = pf.TransferBackend(0)
    stream = torch.cuda.Stream()
    sp = C.c_void_p(stream.cuda_stream)

    def shuffled(n):
        state, perm = 0x9E3779B97F4A7C15, list(range(n))     # the reference's seeded xorshift64 Fisher-Yates
        for i in range(n - 1, 0, -1):
            state ^= (state << 13) & 0xFFFFFFFFFFFFFFFF
            state ^= state >> 7
            state ^= (state << 17) & 0xFFFFFFFFFFFFFFFF
            j = state % (i + 1)
            perm[i], perm[j] = perm[j], perm[i]
        return np.asarray(perm, dtype=np.uint64)

    def descs(layout, n):
        slots = np.arange(n, dtype=np.uint64)
        if layout == "contiguous":
            d_off, h_off = slots * seg, slots * seg
        elif layout == "strided_device":
            d_off, h_off = slots * 2 * seg, slots * seg
        else:
            p = shuffled(n)
            d_off, h_off = p * seg, p * seg
        a = np.zeros((n, 6), dtype=np.uint64)      # device, host, host_device, size, device_allocation, host_allocation
        a[:, 0], a[:, 1], a[:, 2], a[:, 3] = device.data_ptr() + d_off, host + h_off, host_dev + h_off, seg
        return a, d_off // seg, h_off // seg

    def submitters(a, n):
        ptr = a.ctypes.data_as(C.c_void_p)
        calls = C.c_size_t()
        out = {"b200": lambda h2d: N.check((N.lib.pf_backend_h2d if h2d else N.lib.pf_backend_d2h)(
            be._h, C.cast(ptr, C.POINTER(N.CopyDesc)), n, sp))}
        out["reference_direct"] = lambda h2d: ref.pfr_submit_direct(ptr, n, int(h2d), sp, C.byref(calls))
        if has_kernel:
            out["reference_kernel"] = lambda h2d: ref.pfr_submit_kernel(ptr, n, int(h2d), sp)
        return out

    rows, exact = [], True
    for layout in ("contiguous", "strided_device", "shuffled"):
        for n in counts:
            a, d_slots, h_slots = descs(layout, n)
            subs = submitters(a, n)
            # this library's copy is checked once per cell: device fragments == host fragments after H2D
            device.zero_()
            torch.cuda.synchronize()
            subs["b200"](True)
            stream.synchronize()
            got = device.view(-1, seg)[torch.from_numpy(d_slots.astype(np.int64)).to(dev)].cpu().numpy()
            exact = exact and bool(np.array_equal(got, hview.reshape(-1, seg)[h_slots.astype(np.int64)]))
            for direction in ("D2H", "H2D"):
                for name, submit in subs.items():
                    if name == "reference_direct" and layout != "contiguous" and n > 16384:
                        iters_here = 5          # 64 Ki single-fragment copies per submission: keep the run short
                    else:
                        iters_here = iters
                    for _ in range(warm):
                        submit(direction == "H2D")
                        stream.synchronize()
                    t0 = time.perf_counter()
                    for _ in range(iters_here):
                        submit(direction == "H2D")
                        stream.synchronize()
                    secs = time.perf_counter() - t0
                    rows.append({"layout": layout, "blocks": n, "direction": direction, "backend": name,
                                 "avg_ms": round(secs * 1e3 / iters_here, 4),
                                 "GiBps": round(n * seg * iters_here / secs / 2**30, 2)})
    st = be.stats()
    be.close()
    pool.close()
    print(json.dumps({"metric": "transfer_grid_GiBps", "unit": "GiB/s", "higher_is_better": True, "n_gpus": 1,
                      "data": "synthetic", "config": {"workload": "transfer_h2d grid", "fragment_bytes": seg,
                                                      "warmup": warm, "iterations": iters},
                      "bit_exact": exact, "device_status": st["device_status"], "rows": rows}))


def run_pool_coldstart(args):
    """Time to first usable byte of the pinned pool, per allocation strategy (the reference times the same
    thing in pegaflow-core/examples/pinned_alloc_*: `cudaHostAlloc`, `mmap` + parallel pre-touch +
    `cudaHostRegister`, and the same on huge pages, pinned_mem.rs:149-270)."""
    import torch
    import pegaflow_b200 as pf

    torch.cuda.set_device(0)
    torch.cuda.synchronize()
    gib = args.pool_gib
    rows = []
    for name, kw in (("cudaHostAlloc", {}), ("mmap+pretouch+register", {"use_mmap": True}),
                     ("hugepages+register", {"use_mmap": True, "use_hugepages": True})):
        t0 = time.perf_counter()
        try:
            pool = pf.PinnedPool(gib << 30, numa_node=pf.numa_node_of_device(0), **kw)
        except pf.PegaFlowError as e:
            rows.append({"strategy": name, "unavailable": str(e)[:120]})
            continue
        secs = time.perf_counter() - t0
        # the memory must be usable by the copy engine at once: one 1 GiB copy each way
        host, host_dev, handle = pool.alloc(1 << 30)
        d = torch.empty(1 << 30, dtype=torch.uint8, device="cuda")
        be = pf.TransferBackend(0)
        descs, nd = be.make_descs([(d.data_ptr(), host, host_dev, 1 << 30)])
        stream = torch.cuda.Stream()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        be.h2d(descs, nd, stream.cuda_stream)
        b.record(stream)
        b.synchronize()
        rows.append({"strategy": name, "gib": gib, "seconds": round(secs, 3), "GiB_per_s": round(gib / secs, 2),
                     "first_h2d_GBps": round((1 << 30) / 1e6 / a.elapsed_time(b), 1)})
        be.close()
        del d
        pool.release(handle)
        t1 = time.perf_counter()
        pool.close()
        rows[-1]["free_seconds"] = round(time.perf_counter() - t1, 3)
    print(json.dumps({"metric": "pinned_pool_coldstart", "unit": "s", "higher_is_better": False, "n_gpus": 1,
                      "host_cores": os.cpu_count(), "rows": rows}))


def keep_stdout_for_the_json_line():
    """Libraries write to file descriptor 1 on their own (NCCL prints its version there when a communicator is
    created): point descriptor 1 at stderr and keep the original for Python's `print`, so that standard output
    carries the bench line and nothing else."""
    sys.stdout.flush()
    ours = os.fdopen(os.dup(1), "w", buffering=1)
    os.dup2(2, 1)
    sys.stdout = ours


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="llama3.1-8b", choices=list(workloads()))
    ap.add_argument("--route", default="auto", choices=["auto", "staged", "zerocopy"])
    ap.add_argument("--link-ctas", type=int, default=0)
    ap.add_argument("--slot-mib", type=int, default=0)
    ap.add_argument("--slots", type=int, default=0)
    ap.add_argument("--copy-streams", type=int, default=0)
    ap.add_argument("--pack-ctas", type=int, default=0)
    ap.add_argument("--gather-slots", type=int, default=0, help="staging slots one gather launch of a save fills")
    ap.add_argument("--no-kernel-timing", action="store_true", help="diagnostic: no event pairs around kernels")
    ap.add_argument("--contiguous-ids", action="store_true", help="diagnostic: block ids in ascending order")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-cpu-baseline", action="store_true")
    ap.add_argument("--skip-peer", action="store_true", help="N > 1: leave the cross-instance NVLink phase out")
    ap.add_argument("--allow-short-warmup", action="store_true", help="profiling runs only")
    ap.add_argument("--traffic-per-launch", type=float, default=None,
                    help="DRAM bytes per launch of the dominant kernel from an ncu capture (recorded in the line)")
    ap.add_argument("--duplex", action="store_true",
                    help="save and load at the same time (the TP=8 configuration's wording) instead of one after the other")
    ap.add_argument("--peer-local", action="store_true", help="with --peer: source and destination on one GPU")
    ap.add_argument("--peer-layers", type=int, default=64)
    ap.add_argument("--peer-pairs", type=int, default=1,
                    help="with --peer: also run this many GPU i -> GPU pairs+i copies at once (needs 2 x pairs GPUs)")
    ap.add_argument("--peer-push", action="store_true", help="with --peer: run the copy kernel on the source GPU")
    ap.add_argument("--ttft", action="store_true",
                    help="cold / warm time-to-first-token shape through the connector hooks, blocking vs layer-wise")
    ap.add_argument("--ttft-requests", type=int, default=8)
    ap.add_argument("--pool-coldstart", action="store_true", help="time the pinned-pool allocation strategies")
    ap.add_argument("--pool-gib", type=int, default=16)
    ap.add_argument("--transfer-grid", action="store_true",
                    help="the reference's descriptor-level transfer_h2d grid on this library and both reference backends")
    ap.add_argument("--vllm-ttft", action="store_true",
                    help="cold / warm time-to-first-token under a real vLLM engine with this library as its KV connector")
    ap.add_argument("--after-forward", action="store_true",
                    help="with --vllm-ttft: the reference's hook behaviour instead of the layer-wise hooks")
    ap.add_argument("--peer", action="store_true", help="measure the NVLink peer-copy path (one process, two GPUs)")
    ap.add_argument("--pair-overhead", action="store_true",
                    help="event pairs against the kernel's own clock, back to back and inside the pipelines")
    ap.add_argument("--placement-probe", action="store_true",
                    help="time copies into pinned chunks allocated in different ways, alone and with all ranks at once")
    ap.add_argument("--probe-chunk-mib", type=int, default=1024)
    ap.add_argument("--probe-late-chunks", type=int, default=4)
    ap.add_argument("--probe-reps", type=int, default=2)
    ap.add_argument("--probe-hugepages", action="store_true")
    ap.add_argument("--probe-wide-gib", type=int, default=24,
                    help="GiB every rank fills to find chunks far apart in guest-physical memory (0 = skip)")
    args = ap.parse_args()
    world_env = int(os.environ.get("WORLD_SIZE", "1"))
    single_process_mode = args.peer or args.ttft or args.vllm_ttft or args.transfer_grid or args.pool_coldstart or args.pair_overhead
    relaunch = not single_process_mode and args.gpus != world_env and world_env == 1 and args.gpus > 1
    if not relaunch:      # the relaunched ranks do this themselves; their descriptors are this process's
        keep_stdout_for_the_json_line()
    if args.peer:
        run_peer(args)
        return
    if args.ttft:
        run_ttft(args)
        return
    if args.vllm_ttft:
        run_vllm_ttft(args)
        return
    if args.transfer_grid:
        run_transfer_grid(args)
        return
    if args.pool_coldstart:
        run_pool_coldstart(args)
        return
    if args.pair_overhead:
        run_pair_overhead(args)
        return
    if relaunch:
        # convenience: relaunch under torchrun
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29531", os.path.abspath(__file__)] + sys.argv[1:]
        os.execv(sys.executable, cmd)
    rank, world, local = dist_setup(args.gpus)
    try:
        if args.placement_probe:
            run_placement_probe(args, rank, world, local)
        elif args.impl == "reference":
            run_reference(args, rank, world, local)
        else:
            (run_duplex if args.duplex else run_b200)(args, rank, world, local)
    except BaseException:
        # Leave at once: a clean process-group shutdown would wait for the other ranks, and the
        # launcher only stops them when it sees this rank die.
        import traceback

        traceback.print_exc()
        sys.stderr.flush()
        sys.stdout.flush()
        os._exit(1)
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


if __name__ == "__main__":
    main()
