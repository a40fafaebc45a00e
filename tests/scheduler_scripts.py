"""Scripted request lifecycles for the scheduler-side connector.

One interpreter, two users: ``tests/golden/gen_scheduler_traces.py`` runs the scripts on the
reference's ``SchedulerConnector`` (python/pegaflow/connector/scheduler.py) and commits what it
answered; ``tests/test_scheduler_connector.py`` runs them on this repository's mirror and compares.
The fake engine client, request and scheduler-output objects carry only what the connector reads
from vLLM's (`Request.block_hashes`, `KVCacheBlocks.get_block_ids()`, `SchedulerOutput` fields).
"""
from types import SimpleNamespace

BLOCK = 16


def H(i):
    return b"hash-%04d" % i


class FakeClient:
    """Stands in for one TP shard's engine client: a set of stored hashes, prefix queries that hand
    out numbered leases, and a log of everything the connector asked for."""

    def __init__(self, name, ready_cls, loading_cls):
        self.name, self.ready_cls, self.loading_cls = name, ready_cls, loading_cls
        self.store, self.loading, self.live, self.log, self.issued = set(), {}, {}, [], 0
        self.group_store = {}       # storage group id -> hashes whose recurrent state is stored

    def _ready(self, hits, lease, positions):
        answer = self.ready_cls(hits, lease)      # the reference's test stub takes two arguments
        answer.hit_positions = list(positions)
        return answer

    def query_prefetch(self, instance_id, block_hashes, req_id, wait_for_full_prefix=False, group_id=0):
        if group_id != 0:
            # membership: which of the hashes this storage group holds, wherever they are in the query
            held = self.group_store.get(group_id, set())
            positions = [i for i, h in enumerate(block_hashes) if bytes(h) in held]
            if not positions:
                self.log.append(["member-miss", self.name, req_id, group_id, len(block_hashes)])
                return self._ready(0, b"", [])
            self.issued += 1
            lease = b"%s-lease-%03d" % (self.name.encode(), self.issued)
            self.live[lease] = len(positions)
            self.log.append(["member-lease", self.name, req_id, group_id, len(block_hashes), positions, lease.decode()])
            return self._ready(len(positions), lease, positions)
        if self.loading.get(req_id, 0) > 0:
            self.loading[req_id] -= 1
            self.log.append(["loading", self.name, req_id, len(block_hashes)])
            return self.loading_cls()
        n = 0
        for h in block_hashes:
            if bytes(h) not in self.store:
                break
            n += 1
        if n == 0:
            self.log.append(["miss", self.name, req_id, len(block_hashes)])
            return self._ready(0, b"", [])
        self.issued += 1
        lease = b"%s-lease-%03d" % (self.name.encode(), self.issued)
        self.live[lease] = n
        self.log.append(["lease", self.name, req_id, len(block_hashes), n, lease.decode(), bool(wait_for_full_prefix)])
        return self._ready(n, lease, range(n))

    def release(self, lease):
        self.log.append(["release", self.name, bytes(lease).decode()])
        self.live.pop(bytes(lease), None)


class FakeRequest:
    def __init__(self, request_id, hashes, num_tokens):
        self.request_id = request_id
        self.block_hashes = [H(i) for i in hashes]
        self.num_tokens = num_tokens
        self.num_prompt_tokens = num_tokens
        self.num_computed_tokens = 0
        self.prompt_token_ids = list(range(num_tokens))
        self.lora_request = None
        self.cache_salt = None
        self.mm_features = None


class FakeBlockPool:
    """vLLM's GPU block pool as the hybrid save path reads it: the blocks (one per cache group) that
    hold a given block hash locally, or None while some group has none."""

    def __init__(self):
        self.by_hash = {}

    def get_cached_block(self, block_hash, group_ids):
        ids = self.by_hash.get(bytes(block_hash))
        if ids is None:
            return None
        return [SimpleNamespace(block_id=ids[g]) for g in group_ids]


def _groups_of(ids):
    """Block ids as vLLM passes them: a tuple of per-group lists (scripts write one flat list for the
    single-group case)."""
    if ids and isinstance(ids[0], (list, tuple)):
        return tuple(list(g) for g in ids)
    return tuple([list(ids)])


class FakeBlocks:
    """`KVCacheBlocks` as the connector sees it: ids per group, and which blocks already carry a
    hash (the locally computed prefix)."""

    def __init__(self, block_ids, n_cached):
        groups = block_ids if block_ids and isinstance(block_ids[0], (list, tuple)) else [block_ids]
        self._ids = [list(g) for g in groups]
        self.blocks = [[SimpleNamespace(block_hash=(b"x" if i < n_cached else None)) for i in range(len(g))]
                       for g in groups]

    def get_block_ids(self):
        return tuple(self._ids)


def _intent(x):
    out = {"block_ids": [list(g) for g in x.block_ids_by_group]}
    if hasattr(x, "leases"):
        out["leases"] = [bytes(l).decode() for l in x.leases]
        out["num_tokens"] = x.num_tokens
        hold = getattr(x, "recurrent_hold", None)
        if hold is not None:
            out["hold"] = {"leases": [[bytes(l).decode() for l in g] for g in hold.leases],
                           "positions": [[list(p) for p in g] for g in hold.hit_positions], "checkpoint": hold.checkpoint}
    else:
        out["hashes"] = [bytes(h).decode() for h in x.block_hashes]
    return out


def run_script(script, make_connector, ready_cls, loading_cls):
    cfg = dict(block_size=BLOCK, read_enabled=True, wait_for_full_prefix=False, shards=1, recurrent_groups=0)
    cfg.update(script.get("config", {}))
    clients = [FakeClient("shard%d" % i, ready_cls, loading_cls) for i in range(cfg["shards"])]
    conn = make_connector(clients, block_size=cfg["block_size"], read_enabled=cfg["read_enabled"],
                          wait_for_full_prefix=cfg["wait_for_full_prefix"], group_count=1,
                          recurrent_groups=cfg["recurrent_groups"])
    pool = FakeBlockPool()
    if cfg["recurrent_groups"]:
        conn.bind_gpu_block_pool(pool)
    requests, trace = {}, []
    for op in script["ops"]:
        kind, args = op[0], op[1:]
        result = None
        try:
            if kind == "store":
                clients[args[0]].store.update(H(i) for i in args[1])
            elif kind == "evict":
                clients[args[0]].store.difference_update(H(i) for i in args[1])
            elif kind == "gstore":
                clients[args[0]].group_store.setdefault(args[1], set()).update(H(i) for i in args[2])
            elif kind == "pool":
                pool.by_hash.update({H(int(i)): list(ids) for i, ids in args[0].items()})
            elif kind == "computed":
                requests[args[0]].num_computed_tokens = args[1]
            elif kind == "loading":
                clients[args[0]].loading[args[1]] = args[2]
            elif kind == "request":
                requests[args[0]] = FakeRequest(args[0], args[1], args[2])
            elif kind == "grow":
                requests[args[0]].block_hashes.extend(H(i) for i in args[1])
                requests[args[0]].num_tokens = args[2]
            elif kind == "match":
                tokens, load_async = conn.get_num_new_matched_tokens(requests[args[0]], args[1])
                result = [tokens, bool(load_async)]
            elif kind == "alloc":
                req_id, block_ids, n_cached, n_external = args
                blocks = FakeBlocks(block_ids, n_cached) if block_ids is not None else None
                conn.update_state_after_alloc(requests[req_id], blocks, n_external)
                result = "ok"
            elif kind == "step":
                spec = args[0]
                new = [SimpleNamespace(req_id=r, block_ids=(_groups_of(ids) if ids is not None else None),
                                       num_computed_tokens=nc) for r, ids, nc, _n in spec.get("new", [])]
                cached = spec.get("cached", [])
                out = SimpleNamespace(
                    scheduled_new_reqs=new,
                    scheduled_cached_reqs=SimpleNamespace(
                        req_ids=[c[0] for c in cached],
                        new_block_ids=[(_groups_of(c[1]) if c[1] is not None else None) for c in cached],
                        num_computed_tokens=[c[2] for c in cached],
                        resumed_req_ids={c[0] for c in cached if len(c) > 4 and c[4]}),
                    num_scheduled_tokens={**{r: n for r, _i, _c, n in spec.get("new", [])},
                                          **{c[0]: c[3] for c in cached}},
                    preempted_req_ids=set(spec.get("preempted", [])))
                meta = conn.build_connector_meta(out)
                result = {"loads": {k: _intent(v) for k, v in sorted(meta.load_intents.items())},
                          "saves": {k: _intent(v) for k, v in sorted(meta.save_intents.items())},
                          "ready_saves": {k: _intent(v) for k, v in sorted(meta.ready_save_intents.items())},
                          "preempted": sorted(meta.preempted_req_ids)}
            elif kind == "finished":
                held, extra = conn.request_finished(requests[args[0]], _groups_of(args[1]))
                result = [bool(held), extra]
            elif kind == "sent":
                conn.update_connector_output(SimpleNamespace(finished_sending=set(args[0]), finished_recving=None))
            elif kind == "shutdown":
                conn.shutdown()
            else:
                raise ValueError("unknown op " + kind)
        except (RuntimeError, AssertionError) as e:
            result = "error:" + type(e).__name__
        log = []
        for c in clients:
            log.extend(c.log)
            c.log = []
        trace.append({"op": [kind] + [a if not isinstance(a, (set, tuple)) else list(a) for a in args],
                      "result": result, "client_log": log, "live_leases": sorted(l.decode() for c in clients for l in c.live)})
    return trace


def _r(a, b):
    return list(range(a, b))


SCRIPTS = {
    # 56-token prompt (3 full blocks + 8), no cached prefix anywhere: chunked prefill, blocks are saved as
    # they fill, decode completes the fourth block, the request finishes while its last save is pending.
    "cold_prefill_then_decode": {"ops": [
        ("request", "a", _r(0, 3), 56),
        ("match", "a", 0),
        ("alloc", "a", [10, 11, 12, 13], 0, 0),
        ("step", {"new": [["a", [10, 11, 12, 13], 0, 40]]}),
        ("step", {"cached": [["a", None, 40, 16]]}),
        ("grow", "a", [3], 65),
        ("step", {"cached": [["a", [14], 56, 1]]}),
        ("step", {"cached": [["a", None, 57, 1]]}),
        ("step", {"cached": [["a", None, 58, 1]]}),
        ("step", {"cached": [["a", None, 59, 1]]}),
        ("step", {"cached": [["a", None, 60, 1]]}),
        ("step", {"cached": [["a", None, 61, 1]]}),
        ("step", {"cached": [["a", None, 62, 1]]}),
        ("step", {"cached": [["a", None, 63, 1]]}),
        ("step", {"cached": [["a", None, 64, 1]]}),
        ("finished", "a", [10, 11, 12, 13, 14]),
        ("sent", ["a"]),
        ("finished", "a", [10, 11, 12, 13, 14]),
    ]},
    # every block of a 64-token prompt is stored: the hit is clamped so that one token is left to compute
    "warm_full_hit": {"ops": [
        ("store", 0, _r(0, 4)),
        ("request", "w", _r(0, 4), 64),
        ("match", "w", 0),
        ("alloc", "w", [5, 6, 7, 8], 0, 63),
        ("step", {"new": [["w", [5, 6, 7, 8], 63, 1]]}),
        ("grow", "w", [], 65),
        ("step", {"cached": [["w", [9], 64, 1]]}),
        ("finished", "w", [5, 6, 7, 8, 9]),
    ]},
    # two blocks are in the local prefix cache, the store holds the next three of five
    "partial_hit_after_local_prefix": {"ops": [
        ("store", 0, _r(0, 5)),
        ("evict", 0, [0]),
        ("request", "p", _r(0, 6), 100),
        ("match", "p", 0),
        ("store", 0, [0]),
        ("evict", 0, [5]),
        ("match", "p", 32),
        ("alloc", "p", [20, 21, 22, 23, 24, 25, 26], 2, 48),
        ("step", {"new": [["p", [20, 21, 22, 23, 24, 25, 26], 80, 20]]}),
        ("step", {"cached": [["p", None, 100, 1]]}),
        ("finished", "p", [20, 21, 22, 23, 24, 25, 26]),
        ("sent", ["p"]),
    ]},
    # the backend answers Loading twice (a slower tier is fetching), then Ready
    "loading_then_ready": {"config": {"wait_for_full_prefix": True}, "ops": [
        ("store", 0, _r(0, 3)),
        ("request", "l", _r(0, 3), 50),
        ("loading", 0, "l", 2),
        ("match", "l", 0),
        ("match", "l", 0),
        ("match", "l", 0),
        ("match", "l", 0),
        ("alloc", "l", [1, 2, 3, 4], 0, 48),
        ("step", {"new": [["l", [1, 2, 3, 4], 48, 2]]}),
    ]},
    # the request makes local progress while the backend is loading: the Ready that finally arrives
    # belongs to the old query and is released, the next poll starts over
    "identity_drift_while_loading": {"ops": [
        ("store", 0, _r(0, 4)),
        ("request", "d", _r(0, 4), 70),
        ("loading", 0, "d", 1),
        ("match", "d", 0),
        ("match", "d", 16),
        ("match", "d", 16),
        ("alloc", "d", [1, 2, 3, 4, 5], 1, 48),
        ("step", {"new": [["d", [1, 2, 3, 4, 5], 64, 6]]}),
    ]},
    # a cached Ready is reused while the query stays the same, released when it no longer matches,
    # and released at shutdown when nothing consumed it
    "ready_reuse_and_stale_release": {"ops": [
        ("store", 0, _r(0, 4)),
        ("request", "s", _r(0, 4), 80),
        ("match", "s", 0),
        ("match", "s", 0),
        ("match", "s", 32),
        ("request", "t", _r(0, 2), 40),
        ("match", "t", 0),
        ("shutdown",),
    ]},
    # nothing left to query; a miss; a hit whose allocation does not match the lease
    "edge_cases_and_errors": {"ops": [
        ("store", 0, _r(0, 2)),
        ("request", "e1", _r(0, 2), 33),
        ("match", "e1", 32),
        ("request", "e2", _r(7, 9), 40),
        ("match", "e2", 0),
        ("request", "e3", _r(0, 2), 40),
        ("match", "e3", 0),
        ("alloc", "e3", [1, 2, 3], 0, 16),
        ("request", "e4", _r(0, 2), 40),
        ("alloc", "e4", [1, 2, 3], 0, 32),
        ("request", "e5", _r(0, 2), 40),
        ("match", "e5", 0),
        ("alloc", "e5", [1], 0, 32),
        ("request", "e6", _r(0, 2), 40),
        ("step", {"new": [["e6", [4, 5, 6], 0, 40]]}),
    ]},
    # two node-local TP shards: the hit is the prefix both hold, the longer shard is re-leased exactly
    "two_shards_common_prefix": {"config": {"shards": 2}, "ops": [
        ("store", 0, _r(0, 4)),
        ("store", 1, _r(0, 2)),
        ("request", "x", _r(0, 4), 70),
        ("match", "x", 0),
        ("alloc", "x", [1, 2, 3, 4, 5], 0, 32),
        ("step", {"new": [["x", [1, 2, 3, 4, 5], 32, 38]]}),
        ("request", "y", _r(0, 4), 70),
        ("loading", 1, "y", 1),
        ("match", "y", 0),
        ("evict", 1, _r(0, 2)),
        ("match", "y", 0),
    ]},
    # save-only mode: no lookups, saves follow the scheduler's computed-token counts
    "save_only_mode": {"config": {"read_enabled": False}, "ops": [
        ("store", 0, _r(0, 3)),
        ("request", "o", _r(0, 3), 50),
        ("match", "o", 0),
        ("alloc", "o", [1, 2, 3, 4], 0, 0),
        ("step", {"new": [["o", [1, 2, 3, 4], 0, 20]]}),
        ("step", {"cached": [["o", None, 20, 30]]}),
        ("finished", "o", [1, 2, 3, 4]),
        ("sent", ["o"]),
        ("finished", "o", [1, 2, 3, 4]),
    ]},
    # two requests in flight: one warm (loads), one cold (saves), scheduled in the same steps
    "two_requests_interleaved": {"ops": [
        ("store", 0, _r(0, 3)),
        ("request", "u", _r(0, 3), 60),
        ("request", "v", _r(10, 14), 70),
        ("match", "u", 0),
        ("alloc", "u", [1, 2, 3, 4], 0, 48),
        ("match", "v", 0),
        ("alloc", "v", [5, 6, 7, 8, 9], 0, 0),
        ("step", {"new": [["u", [1, 2, 3, 4], 48, 12], ["v", [5, 6, 7, 8, 9], 0, 40]]}),
        ("step", {"cached": [["u", None, 60, 1], ["v", None, 40, 30]]}),
        ("grow", "u", [3], 70),
        ("step", {"cached": [["u", None, 61, 1], ["v", None, 70, 1]]}),
        ("finished", "v", [5, 6, 7, 8, 9]),
        ("step", {"cached": [["u", None, 62, 2]]}),
        ("sent", ["v"]),
        ("finished", "u", [1, 2, 3, 4]),
    ]},
    # a request is dropped while it still holds a Ready lookup (never allocated): the lease goes back
    "finished_before_allocation": {"ops": [
        ("store", 0, _r(0, 2)),
        ("request", "z", _r(0, 2), 40),
        ("match", "z", 0),
        ("finished", "z", []),
        ("request", "z2", _r(0, 2), 40),
        ("loading", 0, "z2", 5),
        ("match", "z2", 0),
        ("finished", "z2", []),
    ]},
    # a long decode: hashes appear one block at a time and are saved as soon as their block is full
    "decode_fills_blocks": {"ops": [
        ("request", "g", _r(0, 1), 20),
        ("match", "g", 0),
        ("alloc", "g", [1, 2], 0, 0),
        ("step", {"new": [["g", [1, 2], 0, 20]]}),
        ("step", {"cached": [["g", None, 20, 6]]}),
        ("step", {"cached": [["g", None, 26, 6]]}),
        ("grow", "g", [1], 33),
        ("step", {"cached": [["g", [3], 32, 6]]}),
        ("step", {"cached": [["g", None, 38, 10]]}),
        ("grow", "g", [2], 49),
        ("step", {"cached": [["g", [4], 48, 1]]}),
        ("finished", "g", [1, 2, 3, 4]),
        ("sent", ["g"]),
        ("finished", "g", [1, 2, 3, 4]),
    ]},
    # a warm request is preempted after its load and resumed later: the loaded prefix is not saved again
    "hit_then_preempt_and_resume": {"ops": [
        ("store", 0, _r(0, 2)),
        ("request", "h", _r(0, 4), 64),
        ("match", "h", 0),
        ("alloc", "h", [1, 2, 3, 4], 0, 32),
        ("step", {"new": [["h", [1, 2, 3, 4], 32, 16]]}),
        ("step", {"preempted": ["h"]}),
        ("match", "h", 0),
        ("alloc", "h", [7, 8, 9, 10], 0, 32),
        ("step", {"cached": [["h", [7, 8, 9, 10], 32, 32, True]]}),
        ("finished", "h", [7, 8, 9, 10]),
    ]},
    # preempted after two blocks were saved, resumed with a fresh block table
    "preempt_and_resume": {"ops": [
        ("request", "r", _r(0, 4), 64),
        ("match", "r", 0),
        ("alloc", "r", [1, 2, 3, 4], 0, 0),
        ("step", {"new": [["r", [1, 2, 3, 4], 0, 32]]}),
        ("step", {"preempted": ["r"]}),
        ("step", {"cached": [["r", [7, 8, 9, 10], 0, 48, True]]}),
        ("step", {"cached": [["r", None, 48, 16]]}),
        ("finished", "r", [7, 8, 9, 10]),
    ]},
}

# ---- hybrid models: one attention cache group and recurrent-state groups ---------------------------------------
# Block ids are written per group ([attention ids, recurrent ids, ...]); the block pool maps a block hash
# to the local block of every group ("pool"); "gstore" puts recurrent checkpoints into a storage group.
HYBRID = {"recurrent_groups": 1}

SCRIPTS.update({
    # nothing cached: blocks are saved only once they were complete before the step and every group's block
    # is in vLLM's block pool; the rest, and the recurrent state after the last full block, at the finish
    "hybrid_cold_saves_from_the_block_pool": {"config": HYBRID, "ops": [
        ("request", "h", _r(0, 3), 56),
        ("match", "h", 0),
        ("alloc", "h", [[10, 11, 12, 13], [30, 31, 32, 33]], 0, 0),
        ("step", {"new": [["h", [[10, 11, 12, 13], [30, 31, 32, 33]], 0, 40]]}),
        ("step", {"cached": [["h", None, 40, 16]]}),
        ("pool", {"0": [10, 30], "1": [11, 31]}),
        ("step", {"cached": [["h", None, 56, 1]]}),
        ("pool", {"2": [12, 32]}),
        ("step", {"cached": [["h", None, 57, 1]]}),
        ("grow", "h", [3], 65),
        ("step", {"cached": [["h", [[14], [34]], 58, 6]]}),
        ("computed", "h", 64),
        ("finished", "h", [[10, 11, 12, 13, 14], [30, 31, 32, 33, 34]]),
        ("step", {}),
        ("sent", ["h"]),
        ("finished", "h", [[10, 11, 12, 13, 14], [30, 31, 32, 33, 34]]),
    ]},
    # attention prefix of four blocks, recurrent checkpoints at positions 1 and 3: the hit ends at 3,
    # the recurrent group loads only the checkpoint's state block
    "hybrid_warm_hit": {"config": HYBRID, "ops": [
        ("store", 0, _r(0, 4)),
        ("gstore", 0, 1, [1, 3]),
        ("request", "w", _r(0, 4), 70),
        ("match", "w", 0),
        ("match", "w", 0),
        ("alloc", "w", [[5, 6, 7, 8, 9], [40, 41, 42, 43, 44]], 0, 64),
        ("step", {"new": [["w", [[5, 6, 7, 8, 9], [40, 41, 42, 43, 44]], 64, 6]]}),
        ("computed", "w", 70),
        ("finished", "w", [[5, 6, 7, 8, 9], [40, 41, 42, 43, 44]]),
    ]},
    # the whole 64-token prompt is stored: one token must be left to compute, which cuts into the last
    # block, so the hit falls back to the checkpoint at position 1
    "hybrid_hit_clamped_to_an_earlier_checkpoint": {"config": HYBRID, "ops": [
        ("store", 0, _r(0, 4)),
        ("gstore", 0, 1, [1, 3]),
        ("request", "c", _r(0, 4), 64),
        ("match", "c", 0),
        ("alloc", "c", [[5, 6, 7, 8], [40, 41, 42, 43]], 0, 32),
        ("step", {"new": [["c", [[5, 6, 7, 8], [40, 41, 42, 43]], 32, 32]]}),
    ]},
    # same, but the only checkpoint is the last block's: nothing usable survives the clamp
    "hybrid_hit_lost_to_the_clamp": {"config": HYBRID, "ops": [
        ("store", 0, _r(0, 4)),
        ("gstore", 0, 1, [3]),
        ("request", "l", _r(0, 4), 64),
        ("match", "l", 0),
        ("alloc", "l", [[5, 6, 7, 8], [40, 41, 42, 43]], 0, 0),
        ("step", {"new": [["l", [[5, 6, 7, 8], [40, 41, 42, 43]], 0, 64]]}),
    ]},
    # an attention prefix without any recurrent checkpoint is a miss, and so is a checkpoint beyond the prefix
    "hybrid_prefix_without_a_checkpoint": {"config": HYBRID, "ops": [
        ("store", 0, _r(0, 3)),
        ("request", "n", _r(0, 5), 100),
        ("match", "n", 0),
        ("gstore", 0, 1, [4]),
        ("match", "n", 0),
        ("gstore", 0, 1, [0]),
        ("match", "n", 0),
        ("alloc", "n", [[1, 2, 3, 4, 5, 6, 7], [11, 12, 13, 14, 15, 16, 17]], 0, 16),
        ("step", {"new": [["n", [[1, 2, 3, 4, 5, 6, 7], [11, 12, 13, 14, 15, 16, 17]], 16, 84]]}),
    ]},
    # the checkpoint lies before the end of the attention prefix: the prefix lease is exchanged for
    # one over exactly the shortened prefix
    "hybrid_shortened_prefix_is_leased_again": {"config": HYBRID, "ops": [
        ("store", 0, _r(0, 4)),
        ("gstore", 0, 1, [1]),
        ("request", "s", _r(0, 5), 90),
        ("match", "s", 0),
        ("alloc", "s", [[1, 2, 3, 4, 5, 6], [11, 12, 13, 14, 15, 16]], 0, 32),
        ("step", {"new": [["s", [[1, 2, 3, 4, 5, 6], [11, 12, 13, 14, 15, 16]], 32, 58]]}),
        ("shutdown",),
    ]},
    # two TP shards and two recurrent groups: the checkpoint has to exist everywhere
    "hybrid_two_shards_two_groups": {"config": {"recurrent_groups": 2, "shards": 2}, "ops": [
        ("store", 0, _r(0, 6)),
        ("store", 1, _r(0, 5)),
        ("gstore", 0, 1, [0, 2, 4]),
        ("gstore", 1, 1, [2, 4]),
        ("gstore", 0, 2, [2, 3, 4]),
        ("gstore", 1, 2, [1, 2]),
        ("request", "t", _r(0, 6), 120),
        ("match", "t", 0),
        ("alloc", "t", [[1, 2, 3, 4, 5, 6, 7, 8], [11, 12, 13, 14, 15, 16, 17, 18], [21, 22, 23, 24, 25, 26, 27, 28]], 0, 48),
        ("step", {"new": [["t", [[1, 2, 3, 4, 5, 6, 7, 8], [11, 12, 13, 14, 15, 16, 17, 18],
                                 [21, 22, 23, 24, 25, 26, 27, 28]], 48, 72]]}),
    ]},
    # a slower tier is loading while the request moves on: the stale answer's prefix and recurrent leases go back
    "hybrid_drift_while_loading": {"config": HYBRID, "ops": [
        ("store", 0, _r(0, 4)),
        ("gstore", 0, 1, [1, 2]),
        ("request", "d", _r(0, 4), 80),
        ("loading", 0, "d", 1),
        ("match", "d", 0),
        ("match", "d", 16),
        ("match", "d", 16),
        ("shutdown",),
    ]},
    # a Ready answer is kept between polls, replaced when the request's position changes, and dropped at the finish
    "hybrid_ready_reuse_and_release": {"config": HYBRID, "ops": [
        ("store", 0, _r(0, 4)),
        ("gstore", 0, 1, [0, 1, 2, 3]),
        ("request", "r", _r(0, 4), 80),
        ("match", "r", 0),
        ("match", "r", 0),
        ("match", "r", 32),
        ("finished", "r", [[1], [2]]),
    ]},
    # refused inputs: a flat block table for a two-group model, a block table shorter than the load, a final
    # recurrent table without the state block after the last full block
    "hybrid_errors": {"config": HYBRID, "ops": [
        ("store", 0, _r(0, 2)),
        ("gstore", 0, 1, [1]),
        ("request", "e", _r(0, 3), 50),
        ("match", "e", 0),
        ("alloc", "e", [1, 2, 3, 4], 0, 32),
        ("match", "e", 0),
        ("alloc", "e", [[1, 2, 3, 4], [11]], 0, 32),
        ("match", "e", 0),
        ("alloc", "e", [[1, 2, 3, 4], [11, 12, 13, 14]], 0, 32),
        ("step", {"new": [["e", [[1, 2, 3, 4], [11, 12, 13, 14]], 32, 18]]}),
        ("computed", "e", 50),
        ("finished", "e", [[1, 2, 3, 4], [11, 12, 13]]),
        ("finished", "e", [[1, 2, 3, 4], [11, 12, 13, 14]]),
    ]},
})
