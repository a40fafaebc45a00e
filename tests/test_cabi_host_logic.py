"""CPU-only checks of the product library: it loads, exports every symbol the header declares,
and its pure host logic (layout arithmetic, page layout, allocator unit, LoadState) agrees with
the reference's known-answer tests and with the oracle.  No compute call needs a GPU here."""
import ctypes as C
import os
import re

import pytest

import pegaflow_b200 as pf
from pegaflow_b200 import _native as N
from oracle import pf_oracle as po

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "pegaflow_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pf_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = _declared_symbols()
    assert len(names) >= 50
    for name in names:
        assert hasattr(N.lib, name), f"{name} is declared in include/pegaflow_b200.h but not exported"
    assert N.lib.pf_abi_version() == 1


def _layout(case):
    out = N.Layout()
    a = case["new"]
    st = N.lib.pf_layout_init(C.byref(out), a[0], a[1], a[2], a[3], a[4], a[5], case.get("block_stride", 0),
                              case.get("ssd_padding", 0))
    return st, out


def test_layout_known_answers_through_the_c_abi(kats):
    for case in kats["layout"]["ok"]:
        st, lay = _layout(case)
        assert st == 0, (case["name"], N.lib.pf_last_error())
        if "split" in case:
            assert bool(lay.split) == case["split"]
        for idx, want in case.get("copies", {}).items():
            addr, nbytes, n = (C.c_uint64 * 2)(), (C.c_size_t * 2)(), C.c_int()
            assert N.lib.pf_layout_block_copies(C.byref(lay), int(idx), addr, nbytes, C.byref(n)) == 0
            assert [[addr[i], nbytes[i]] for i in range(n.value)] == want, case["name"]
        for idx in case.get("out_of_range", []):
            addr, nbytes, n = (C.c_uint64 * 2)(), (C.c_size_t * 2)(), C.c_int()
            assert N.lib.pf_layout_block_copies(C.byref(lay), idx, addr, nbytes, C.byref(n)) == 3
            assert b"out of range" in N.lib.pf_last_error()
        if "padded_segment_bytes" in case:
            assert lay.padded_segment_bytes == case["padded_segment_bytes"]
            assert lay.padded_segment_bytes * lay.segments == case["padded_block_bytes"]
    for case in kats["layout"]["reject"]:
        st, _ = _layout(case)
        assert st == 3, case["name"]
        msg = N.lib.pf_last_error().decode()
        assert case["contains"] in msg and msg.startswith("invalid argument: "), (case["name"], msg)


def test_layout_matches_oracle_on_random_geometries():
    import numpy as np

    rng = np.random.default_rng(3)
    agree = 0
    for _ in range(3000):
        seg = int(rng.choice([64, 100, 512, 1024, 4096, 8848]))
        nb = int(rng.integers(1, 40))
        segs = int(rng.choice([1, 2, 2, 3]))
        kv = int(rng.choice([0, seg // 2, seg, seg * 2, seg * nb, seg * nb + 48, seg * (nb // 2) + 7]))
        stride = int(rng.choice([0, 0, seg, seg * 2, seg * segs, seg * segs + 16, seg - 1]))
        size = int(rng.choice([seg * segs * nb, seg * segs * nb * 3, 1 << 30, seg]))
        args = (0x7000, size, nb, seg, kv, segs)
        out = N.Layout()
        st = N.lib.pf_layout_init(C.byref(out), *args, stride, 512)
        try:
            o = po.KVCacheLayout(*args)
            if stride:
                o.with_block_stride(stride)
            o.with_ssd_padding(512)
            err = None
        except po.OracleError as e:
            err = str(e)
        if err is None:
            assert st == 0, (args, stride, N.lib.pf_last_error())
            for f in ("block_stride_bytes", "segment_bytes", "segments", "padded_segment_bytes", "split", "kv_stride_bytes"):
                assert getattr(out, f) == getattr(o.c, f), (f, args, stride)
            agree += 1
        else:
            assert st == 3 and N.lib.pf_last_error().decode() == "invalid argument: " + err, (args, stride, err)
    assert agree > 200


def test_page_layout_and_unit_size_through_the_c_abi(kats):
    SZ = C.c_size_t
    for case in kats["page_layout"]["ok"] + kats["page_layout"]["reject"]:
        sets = case["sets"]
        offs, items = [0], []
        for s in sets:
            items += s
            offs.append(len(items))
        n = case["n_layers"]
        shard, loff, lbytes, pages, nsh = (SZ * n)(), (SZ * n)(), (SZ * n)(), (SZ * len(sets))(), SZ()
        st = N.lib.pf_build_page_layout((SZ * len(offs))(*offs), (SZ * len(items))(*items), len(sets), n,
                                        (SZ * n)(*case["padded"]), shard, loff, lbytes, pages, C.byref(nsh))
        if "contains" in case:
            assert st == 3 and case["contains"] in N.lib.pf_last_error().decode()
        else:
            assert st == 0
            assert list(shard) == case["layer_shard"] and list(loff) == case["layer_offsets"]
            assert list(lbytes) == case["layer_bytes"] and list(pages[: nsh.value]) == case["shard_page_sizes"]
    for case in kats["allocator"]["unit_size"]:
        assert N.lib.pf_pool_unit_size(case["pool"], case["hint"]) == case["unit"]


def test_load_state_segment_is_bit_compatible(kats):
    ls = kats["load_state"]
    state = pf.PyLoadState()
    name = state.shm_name()
    assert name.startswith(ls["name_prefix"]) and len(name) == len(ls["name_prefix"]) + 32
    raw = open("/dev/shm/" + name, "rb").read()
    assert raw == po.load_state_image(0) and len(raw) == ls["mapping_bytes"]
    other = pf.PyLoadState(attach_to=name)
    state.set_completed()
    assert other.get_state() == ls["success"] and po.parse_load_state(open("/dev/shm/" + name, "rb").read()) == 1
    other.set_error()
    assert state.get_state() == ls["error"]
    # an image written by the other side (the oracle stands in for the reference) attaches as well
    foreign = "pega_load_" + "0" * 31 + "f"
    with open("/dev/shm/" + foreign, "wb") as f:
        f.write(po.load_state_image(1))
    try:
        assert pf.PyLoadState(attach_to=foreign).get_state() == 1
        with open("/dev/shm/" + foreign, "wb") as f:
            f.write(b"\0")
        with pytest.raises(pf.PegaflowInternal, match="too small"):
            pf.PyLoadState(attach_to=foreign)
        bad = bytearray(po.load_state_image(0))
        bad[8:12] = (0xDEADBEEF).to_bytes(4, "little")
        with open("/dev/shm/" + foreign, "wb") as f:
            f.write(bytes(bad))
        with pytest.raises(pf.PegaflowInternal, match="invalid LoadState header"):
            pf.PyLoadState(attach_to=foreign)
    finally:
        os.unlink("/dev/shm/" + foreign)
    del other
    del state
    assert not os.path.exists("/dev/shm/" + name), "the creator unlinks its segment"
    with pytest.raises(pf.PegaflowInternal, match="failed to open shared memory"):
        pf.PyLoadState(attach_to="pega_load_missing")


def test_no_gpu_means_loud_failure_not_a_fallback():
    """Without a CUDA device nothing pretends to work: engine, backend and pool refuse to start."""
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    for make in (lambda: pf.PegaEngine(1 << 20), lambda: pf.TransferBackend(0), lambda: pf.PinnedPool(1 << 20)):
        with pytest.raises(pf.PegaFlowError):
            make()


def test_connector_layout_inference_matches_reference_fixture():
    """The product's host mirror of worker.py:65-151 against outputs of the reference itself."""
    import json

    from pegaflow_b200.connector import infer_kv_cache_registration, resolve_transfer_backend

    class T:
        def __init__(self, shape, stride, es):
            self.shape, self._stride, self._es = tuple(shape), tuple(stride), es

        def stride(self):
            return self._stride

        def element_size(self):
            return self._es

    with open(os.path.join(ROOT, "tests", "golden", "kv_layout_inference.json")) as f:
        cases = json.load(f)["cases"]
    for c in cases:
        t = T(c["shape"], c["stride"], c["element_size"])
        kw = dict(is_mla=c["is_mla"], is_recurrent_state=c["is_recurrent_state"])
        if "error" in c:
            with pytest.raises(ValueError) as ei:
                infer_kv_cache_registration(t, c["logical_block_size"], **kw)
            assert str(ei.value) == c["error"]
        else:
            info = infer_kv_cache_registration(t, c["logical_block_size"], **kw)
            assert {k: getattr(info, k) for k in c["result"]} == c["result"], c
    assert resolve_transfer_backend(True, None) == "kernel" and resolve_transfer_backend(False, None) == "direct"
    assert resolve_transfer_backend(True, "direct") == "direct"
    with pytest.raises(ValueError, match="Unsupported pegaflow.transfer_backend"):
        resolve_transfer_backend(False, "nvlink")


# ---- worker connector: a load that cannot be submitted (python/tests/test_connector_fault_tolerance.py:170-333) ----
class _RejectingClient:
    def __init__(self, mode):
        self.mode, self.load_calls, self.released = mode, 0, []

    def load(self, *args):
        self.load_calls += 1
        if self.mode == "exception":
            raise ConnectionError("server gone")
        return False, "load refused"

    def release(self, lease):
        self.released.append(bytes(lease))


@pytest.mark.parametrize("mode", ["ok_false", "exception"])
def test_worker_reports_a_rejected_load_instead_of_raising(mode):
    from pegaflow_b200.connector import PegaWorkerConnector

    client = _RejectingClient(mode)
    worker = PegaWorkerConnector(client, None, instance_id="i", namespace="n", device_id=0, block_size=16)
    worker.registered_layers = ["layer"]
    worker.start_load_kv([("r1", b"lease-r1", [1])])           # must not raise
    worker.start_load_kv([("r2", b"lease-r2", [2, None, 3])])
    assert client.load_calls == 2 and client.released == [b"lease-r1", b"lease-r2"]
    assert worker.get_block_ids_with_load_errors() == {1, 2, 3}
    assert worker.get_block_ids_with_load_errors() == set()      # drained by the first call
    done, failed = worker.get_finished()
    assert done == [] and failed == ["r1", "r2"]                 # reported, so that nothing stays parked
    assert worker.get_finished() == ([], [])


class _RecordingClient:
    def __init__(self):
        self.saves = []

    def save(self, instance_id, tp_rank, pp_rank, device_id, saves):
        self.saves.append([(n, list(i), list(h)) for n, i, h in saves])
        return True, ""

    def flush_saves(self):
        return True, ""


def test_page_first_saves_are_striped_over_tp_ranks():
    """worker.py:982-1005: under page-first every rank holds all layers of a block, so rank r saves the
    blocks with id % tp_size == r (all their layers); the stripes are disjoint and complete."""
    from pegaflow_b200.connector import PegaWorkerConnector

    ids = [0, 4, 5, 6, 7, 9, 12, 13]
    hashes = [b"h%d" % i for i in ids]
    seen = []
    for rank in range(4):
        client = _RecordingClient()
        w = PegaWorkerConnector(client, None, instance_id="i", namespace="n", device_id=rank, block_size=64, tp_rank=rank,
                                tp_size=4, world_size=4, is_mla=True)
        assert w.page_first
        w.wait_for_save([("layer_a", ids, hashes), ("layer_b", ids, hashes)])
        (batch,) = client.saves
        assert batch[0][1:] == batch[1][1:]                       # every layer of the stripe
        assert all(b % 4 == rank and b != 0 for b in batch[0][1])    # block 0 is vLLM's null block
        assert batch[0][2] == [b"h%d" % b for b in batch[0][1]]
        seen += batch[0][1]
    assert sorted(seen) == [b for b in ids if b != 0]
    # layer-first (non-MLA) workers save everything themselves
    client = _RecordingClient()
    w = PegaWorkerConnector(client, None, instance_id="i", namespace="n", device_id=1, block_size=16, tp_rank=1, tp_size=4,
                            world_size=4)
    w.wait_for_save([("layer_a", ids, hashes)])
    assert client.saves[0][0][1] == [b for b in ids if b != 0]


def test_preemption_flushes_queued_layer_saves():
    from pegaflow_b200.connector import PegaWorkerConnector

    class Client(_RecordingClient):
        flushed = 0

        def save_async(self, *a):
            return True, ""

        def flush_saves(self):
            Client.flushed += 1
            return True, ""

    w = PegaWorkerConnector(Client(), None, instance_id="i", namespace="n", device_id=0, block_size=16)
    w.handle_preemptions({"r"})
    assert Client.flushed == 0                       # nothing queued: nothing to wait for
    w.save_kv_layer("layer", [3, 4], [b"a", b"b"], 0)
    w.handle_preemptions(set())
    assert Client.flushed == 0                       # nobody was preempted
    w.handle_preemptions({"r"})
    assert Client.flushed == 1
    w.handle_preemptions({"r"})
    assert Client.flushed == 1


def test_ipc_entry_points_reject_bad_arguments_without_a_gpu():
    import ctypes as C

    from pegaflow_b200 import _native as N

    region = N.IpcRegion()
    assert N.lib.pf_ipc_export(0, 4096, C.byref(region)) == 3            # invalid argument
    assert b"null pointer or empty region" in N.lib.pf_last_error()
    assert N.lib.pf_ipc_export(0x1000, 0, C.byref(region)) == 3
    assert N.lib.pf_ipc_close(C.byref(region)) == 3
    assert b"not open" in N.lib.pf_last_error()
    assert N.lib.pf_ipc_open(None, None, None) == 3
    assert C.sizeof(N.IpcRegion) == 96


def test_python_client_surface_matches_the_reference_stub():
    """A caller written against the reference's native module (python/pegaflow/pegaflow.pyi) finds
    the same methods with the same parameter order here.  The fixture is that stub's surface, read
    with `ast` by tests/golden/gen_client_surface.py.  Two differences are intended: the client is
    built around an engine instead of an endpoint, and register_context_batch takes the tensors (or
    pickled IPC wrappers) in the position of `wrapper_bytes_list`."""
    import inspect
    import json

    golden = json.load(open(os.path.join(ROOT, "tests", "golden", "engine_client_surface.json")))["classes"]
    mine = {"EngineRpcClient": pf.InProcEngineClient, "PyLoadState": pf.PyLoadState, "QueryReady": pf.QueryReady,
            "QueryLoading": pf.QueryLoading}
    renamed = {("EngineRpcClient", "register_context_batch", "wrapper_bytes_list"): "tensors"}
    for cls_name, spec in golden.items():
        cls = mine[cls_name]
        for method, params in spec["methods"].items():
            if method == "__init__" and cls_name in ("EngineRpcClient", "PyLoadState"):
                continue   # constructed from an engine / optionally attached to an existing segment
            assert hasattr(cls, method), f"{cls_name}.{method} is missing"
            sig = inspect.signature(getattr(cls, method))
            got = [(p.name, p.default is not inspect.Parameter.empty) for p in sig.parameters.values()
                   if p.name != "self" and p.kind not in (p.VAR_POSITIONAL, p.VAR_KEYWORD)]
            want = [(renamed.get((cls_name, method, name), name), has_default) for name, has_default in params]
            assert got[:len(want)] == want, f"{cls_name}.{method}: {got} != {want}"
            assert all(d for _, d in got[len(want):]), f"{cls_name}.{method}: extra parameters must be optional"
        for field in spec["fields"]:
            assert field in getattr(cls, "__dataclass_fields__", {}) or hasattr(cls, field), f"{cls_name}.{field}"


def test_a_load_that_never_completes_times_out_and_its_blocks_are_reported(monkeypatch):
    """worker.py:454-507: a load still pending after LOAD_TIMEOUT_SECONDS is handed back as failed and
    its destination blocks are reported invalid; PEGA_LOAD_TIMEOUT_SECONDS is clamped to 30 s."""
    from pegaflow_b200 import connector
    from pegaflow_b200.connector import PegaWorkerConnector

    class Client(_RecordingClient):
        def load(self, *a):
            return True, ""          # accepted, and then nothing ever sets the state

    w = PegaWorkerConnector(Client(), None, instance_id="i", namespace="n", device_id=0, block_size=16)
    w.registered_layers = ["layer"]
    w.start_load_kv([("req-a", b"L" * 16, [4, None, 9])])
    assert w.get_finished() == ([], []) and w.available
    w._pending_loads[0].started -= w.LOAD_TIMEOUT_SECONDS + 1
    assert w.get_finished() == ([], ["req-a"])
    assert w.get_block_ids_with_load_errors() == {4, 9}
    assert not w.available and w.load_history[-1][1:] == (2, False)
    assert w.get_finished() == ([], [])
    # a load that completes in time is unaffected
    w.start_load_kv([("req-b", b"M" * 16, [5])])
    w._pending_loads[0].state.set_completed()
    assert w.get_finished() == (["req-b"], []) and w.load_history[-1][1:] == (1, True)
    for raw, want in [(None, 120), ("45", 45), ("5", 30), ("abc", 120), ("-1", 30)]:
        if raw is None:
            monkeypatch.delenv("PEGA_LOAD_TIMEOUT_SECONDS", raising=False)
        else:
            monkeypatch.setenv("PEGA_LOAD_TIMEOUT_SECONDS", raw)
        assert connector._load_timeout_seconds() == want


def test_service_state_recovers_once_the_health_probe_succeeds():
    """state_manager.py:47-92: unavailable after a failure, a background probe asks health() and the first
    healthy answer (exceptions and unhealthy answers are skipped) makes the service available again."""
    import time

    from pegaflow_b200.connector import PegaWorkerConnector, ServiceStateManager

    class Client(_RecordingClient):
        answers = [RuntimeError("connection refused"), (False, "starting"), (True, "ok")]
        asked = 0

        def health(self):
            Client.asked += 1
            a = Client.answers.pop(0)
            if isinstance(a, Exception):
                raise a
            return a

        def load(self, *a):
            return False, "engine restarting"

        def release(self, lease):
            pass

    client = Client()
    sm = ServiceStateManager(client, health_check_interval=0.02)
    w = PegaWorkerConnector(client, None, instance_id="i", namespace="n", device_id=0, block_size=16, state_manager=sm)
    w.registered_layers = ["layer"]
    assert w.available
    w.start_load_kv([("req", b"L" * 16, [7])])          # rejected: leases back, blocks invalid, service marked
    assert sm.last_reason == "load rpc failed: engine restarting"
    assert w.get_finished() == ([], ["req"]) and w.get_block_ids_with_load_errors() == {7}
    sm.mark_unavailable("second reason is ignored while unavailable")
    assert sm.last_reason.startswith("load rpc failed")
    deadline = time.time() + 5
    while not sm.is_available() and time.time() < deadline:
        time.sleep(0.01)
    assert sm.is_available() and Client.asked == 3
    w.registered_layers = []
    w.unregister()          # also stops the probe thread


def test_page_layout_and_unit_size_match_the_oracle_on_random_topologies():
    """Random worker layer sets (disjoint shards, identical replicas, overlapping or empty sets that
    must be refused) through the product's C ABI and through the oracle: same layout or both refuse."""
    import numpy as np

    rng = np.random.default_rng(11)
    SZ = C.c_size_t
    agreed_ok = agreed_reject = 0
    for _ in range(300):
        n = int(rng.integers(1, 12))
        kind = rng.choice(["split", "replicas", "random"])
        if kind == "split":
            cuts = sorted(set(rng.integers(1, n, size=int(rng.integers(0, 3))).tolist())) if n > 1 else []
            edges = [0] + cuts + [n]
            sets = [list(range(a, b)) for a, b in zip(edges, edges[1:])]
            sets = [sets[i] for i in rng.permutation(len(sets))] * int(rng.integers(1, 3))
        elif kind == "replicas":
            sets = [list(range(n))] * int(rng.integers(1, 4))
        else:
            sets = [sorted(set(rng.integers(0, n + 1, size=int(rng.integers(0, n + 1))).tolist()))
                    for _ in range(int(rng.integers(1, 4)))]
        padded = (rng.integers(1, 40, size=n) * 512).tolist()
        offs, items = [0], []
        for s in sets:
            items += s
            offs.append(len(items))
        shard, loff, lbytes, pages, nsh = (SZ * n)(), (SZ * n)(), (SZ * n)(), (SZ * len(sets))(), SZ()
        st = N.lib.pf_build_page_layout((SZ * len(offs))(*offs), (SZ * max(1, len(items)))(*items), len(sets), n,
                                        (SZ * n)(*padded), shard, loff, lbytes, pages, C.byref(nsh))
        try:
            want = po.build_page_layout(sets, n, padded)
        except po.OracleError:
            assert st == 3, f"oracle refuses {sets} over {n} layers, the library accepted it"
            agreed_reject += 1
            continue
        assert st == 0, f"oracle accepts {sets} over {n} layers, the library said: {N.lib.pf_last_error().decode()}"
        assert list(shard) == want["layer_shard"] and list(loff) == want["layer_offsets"]
        assert list(lbytes) == want["layer_bytes"] and list(pages[: nsh.value]) == want["shard_page_sizes"]
        agreed_ok += 1
    assert agreed_ok >= 50 and agreed_reject >= 20, (agreed_ok, agreed_reject)
    for _ in range(300):
        pool = int(rng.integers(1, 1 << 46))
        hint = int(rng.choice([0, 1, 511, 512, 513, 4096, 73728, int(rng.integers(1, 1 << 24))]))
        assert N.lib.pf_pool_unit_size(pool, hint) == po.pool_unit_size(pool, hint or None)


def test_engine_entry_points_reject_a_null_engine_without_a_gpu():
    """Every engine-level call added beside the reference's own (instance listing, namespace, cache clean-up,
    metrics, phase times) checks its arguments before it touches anything: InvalidArgument, message kept."""
    buf, need = C.create_string_buffer(16), N.sz()
    assert N.lib.pf_engine_list_instances(None, buf, len(buf), C.byref(need)) == 3
    assert b"null argument" in N.lib.pf_last_error()
    assert N.lib.pf_engine_unregister_all_instances(None, buf, len(buf), C.byref(need)) == 3
    assert N.lib.pf_engine_instance_namespace(None, b"x", buf, len(buf), C.byref(need)) == 3
    assert N.lib.pf_engine_cleanup_memory_cache(None, C.byref(N.CacheCleanupStats())) == 3
    assert N.lib.pf_engine_get_metrics(None, C.byref(N.EngineMetrics())) == 3
    assert N.lib.pf_engine_get_phase_times(None, C.byref(N.PhaseTimes())) == 3
    assert N.lib.pf_engine_phase_name(-1) is None and N.lib.pf_engine_phase_name(N.PHASE_COUNT) is None
    assert N.lib.pf_engine_phase_name(0) == b"save.resolve_metadata"
