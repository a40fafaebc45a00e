"""Scenarios for the TP-shard query client, shared by the fixture generator (which runs them on the
reference's TpShardQueryClient) and the test (which runs them on this package's ShardQuery): scripted
shard answers, and a record of the outcome and of every call the client made to the shards."""
import random


class ScriptedShard:
    """One shard's engine client: answers query_prefetch from a script, logs every call."""

    def __init__(self, index, script, log, ready_cls, loading_cls, failing_releases=()):
        self.index, self.script, self.log = index, list(script), log
        self.ready_cls, self.loading_cls, self.failing_releases = ready_cls, loading_cls, set(failing_releases)

    def query_prefetch(self, instance_id, block_hashes, req_id=None, wait_for_full_prefix=False, group_id=0):
        self.log.append(["query", self.index, len(block_hashes), req_id, bool(wait_for_full_prefix), group_id])
        step = self.script.pop(0) if self.script else ["ready", 0, "", []]
        kind = step[0]
        if kind == "loading":
            return self.loading_cls()
        if kind == "raise":
            raise ConnectionError(step[1])
        _, hits, lease, positions = step
        answer = self.ready_cls(hits, lease.encode())     # the reference's test stub takes two arguments
        answer.hit_positions = list(positions)
        return answer

    def release(self, lease):
        self.log.append(["release", self.index, lease.decode()])
        if lease.decode() in self.failing_releases:
            raise ConnectionError("release failed")


def _outcome(fn):
    try:
        return {"ok": fn()}
    except Exception as e:     # the type is part of the contract: record it
        return {"error": [type(e).__name__, str(e)]}


def scenarios(rng):
    """(kind, n_hashes, per-shard scripts, leases whose release fails, group id)."""
    out = []
    for _ in range(70):
        n_shards = rng.choice([1, 2, 2, 3])
        n_hashes = rng.choice([0, 1, 4, 6])
        kind = rng.choice(["prefix", "prefix", "membership"])
        scripts = []
        for s in range(n_shards):
            roll = rng.random()
            if roll < 0.12:
                first = ["loading"]
            elif roll < 0.2:
                first = ["raise", f"shard {s} unreachable"]
            else:
                hits = rng.choice([0, n_hashes, n_hashes, max(0, n_hashes - 2), n_hashes + 1, 2])
                lease = "" if rng.random() < 0.1 else f"lease-{s}-a"
                if kind == "membership":
                    pool = list(range(n_hashes + (1 if rng.random() < 0.15 else 0)))
                    positions = sorted(rng.sample(pool, min(len(pool), hits))) if rng.random() > 0.1 else []
                else:
                    positions = []
                first = ["ready", hits, lease, positions]
            script = [first]
            if kind == "prefix":     # the follow-up query for exactly the common prefix
                roll = rng.random()
                if roll < 0.15:
                    script.append(["loading"])
                elif roll < 0.25:
                    script.append(["raise", f"shard {s} dropped"])
                else:
                    script.append(["ready", rng.choice(["common", "common", "common", 1, 0]),
                                   "" if rng.random() < 0.1 else f"lease-{s}-b", []])
            scripts.append(script)
        failing = [f"lease-{s}-a" for s in range(n_shards) if rng.random() < 0.1]
        out.append([kind, n_hashes, scripts, failing, rng.choice([1, 2])])
    return out


def run_all(make_client, ready_cls, loading_cls, seed=77):
    """`make_client(shards)` returns the object under test; its `query` answer is normalised with
    `normalise_query` by the caller's adapter (see the generator and the test)."""
    results = []
    for kind, n_hashes, scripts, failing, group_id in scenarios(random.Random(seed)):
        log = []
        firsts = [sc[0] for sc in scripts if sc[0][0] == "ready"]
        ready_first = len(firsts) == len(scripts)
        common = min((sc[0][1] for sc in scripts), default=0) if ready_first else 0
        shards = []
        for i, sc in enumerate(scripts):
            sc = [list(step) for step in sc]
            for step in sc:
                if step[0] == "ready" and step[1] == "common":
                    step[1] = common
            shards.append(ScriptedShard(i, sc, log, ready_cls, loading_cls, failing))
        client = make_client(tuple(shards))
        hashes = [b"h%d" % i for i in range(n_hashes)]
        if kind == "prefix":
            outcome = _outcome(lambda: client.prefix("inst", hashes, "req", False))
        else:
            outcome = _outcome(lambda: client.membership("inst", hashes, "req", group_id))
        results.append({"kind": kind, "n_hashes": n_hashes, "scripts": scripts, "outcome": outcome, "log": log})
    return results
