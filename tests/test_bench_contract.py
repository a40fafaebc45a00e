"""bench.py's `roofline` object keeps the keys the measurement contract names, whichever legs ran:
the kernel-alone leg puts its figure at the top level and moves the in-pipeline figures below it.
Pure host logic on made-up counters; no GPU."""
import importlib.util
import os
from types import SimpleNamespace

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
bench = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(bench)

REQUIRED = {"bound", "achieved", "peak", "unit", "frac", "traffic"}
ARGS = SimpleNamespace(traffic_per_launch=None)


def _stats(launches, ms, nbytes, dev_n=0, dev_ms=0.0, link=(0, 0.0, 0)):
    return {"pack_kernel_launches": launches, "pack_kernel_ms": ms, "pack_kernel_bytes": nbytes,
            "pack_kernel_device_launches": dev_n, "pack_kernel_device_ms": dev_ms,
            "link_kernel_launches": link[0], "link_kernel_ms": link[1], "link_kernel_bytes": link[2]}


def test_roofline_from_pipeline_counters_only():
    zero = _stats(0, 0.0, 0)
    after = _stats(100, 4.0, 100 * 40 << 20, dev_n=100, dev_ms=0.75)
    r = bench.build_roofline([(zero, after)], ARGS)
    assert REQUIRED <= set(r) and r["bound"] == "hbm" and r["unit"] == "GB/s"
    assert r["launches"] == 100 and r["algorithmic_bytes_per_launch"] == 40 << 20
    assert abs(r["achieved"] - (100 * (40 << 20)) / 1e6 / 4.0) < 0.1
    assert abs(r["frac"] - r["achieved"] / r["peak"]) < 1e-3
    assert r["device_clock"]["avg_launch_us"] == 7.5
    assert r["traffic"] == round((40 << 20) / 2 * (8.398336 / 8.388608))   # one DRAM read per payload byte


def test_roofline_headline_is_the_kernel_alone_when_that_leg_ran():
    zero = _stats(0, 0.0, 0)
    after = _stats(100, 4.0, 100 * 40 << 20, dev_n=100, dev_ms=0.75)
    alone = {"ms": 16.0, "launches": 1536, "payload": 1536 * (20 << 20), "passes": 3, "inputs_exceed_l2": True}
    r = bench.build_roofline([(zero, after)], ARGS, alone)
    assert REQUIRED <= set(r)
    assert r["launches"] == 1536 and r["algorithmic_bytes_per_launch"] == 40 << 20
    assert abs(r["achieved"] - 2 * alone["payload"] / 1e6 / 16.0) < 0.1
    assert abs(r["frac"] - r["achieved"] / r["peak"]) < 1e-3
    assert "gather_layers" in r["how"] and r["inputs_exceed_l2"] is True
    # per launch of the headline leg: the reads of the payload plus the write-backs seen during a launch
    assert r["traffic"] == round((20 << 20) * (bench.SAVE_LAUNCH_DRAM_MB / 62.914560))
    assert (20 << 20) < r["traffic"] < r["algorithmic_bytes_per_launch"]
    inner = r["in_pipeline"]
    assert inner["launches"] == 100 and abs(inner["avg_launch_us"] - 40.0) < 1e-6
    assert inner["device_clock"]["frac"] > inner["frac"]
    assert "device_clock" not in r and "note" not in r


def test_roofline_of_the_zero_copy_route_reports_the_link_kernel():
    zero = _stats(0, 0.0, 0)
    after = _stats(0, 0.0, 0, link=(64, 200.0, 10 << 30))
    r = bench.build_roofline([(zero, after)], ARGS)
    assert REQUIRED <= set(r) and r["launches"] == 64 and "PCIe" in r["note"]


def test_sweep_chunk_reports_where_it_lies_and_releases_its_mapping():
    w = bench.WideChunk(8 << 20)
    assert w.addr % 4096 == 0 and w.view[0] == 1 and w.view[4096] == 1 and w.view[1] == 0
    assert w.frames_gib == sorted(w.frames_gib)            # empty where the kernel hides page frames
    assert (w.median_gib in w.frames_gib) if w.frames_gib else w.median_gib == -1.0
    w.close()
    assert w.view is None and w.map.closed


def test_standard_output_is_kept_for_the_json_line():
    """What a library writes to file descriptor 1 on its own (NCCL's version banner) must not share standard
    output with the bench line."""
    import subprocess
    import sys

    code = ("import importlib.util, os\n"
            f"spec = importlib.util.spec_from_file_location('b', {os.path.join(ROOT, 'bench.py')!r})\n"
            "b = importlib.util.module_from_spec(spec); spec.loader.exec_module(b)\n"
            "b.keep_stdout_for_the_json_line()\n"
            "os.write(1, b'library banner\\n')\n"
            "print('{\"metric\": 1}')\n")
    p = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120)
    assert p.returncode == 0 and p.stdout == '{"metric": 1}\n' and p.stderr.endswith("library banner\n")
