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


def hybrid_scenarios(rng):
    """Hybrid lookups: per shard the attention prefix answer, one membership answer per recurrent
    storage group, then the answer to the exact re-lease of a shortened prefix.  Most scripts are
    well-formed so that the success paths are reached; some break at each stage."""
    out = []
    for _ in range(80):
        n_shards, n_groups, n_hashes = rng.choice([1, 2]), rng.choice([1, 2]), rng.choice([4, 6, 8])
        prefix = rng.choice([n_hashes, n_hashes, n_hashes, n_hashes - 1, 2, 0])
        positions = [[sorted(rng.sample(range(n_hashes), rng.choice([0, 1, n_hashes // 2, n_hashes - 1, n_hashes, n_hashes])))
                      for _ in range(n_shards)] for _ in range(n_groups)]
        usable = None
        for group in positions:
            for shard_positions in group:
                inside = {p for p in shard_positions if p < prefix}
                usable = inside if usable is None else usable & inside
        reconciled = max(usable) + 1 if usable else 0
        scripts = []
        for s in range(n_shards):
            roll = rng.random()
            script = [["loading"] if roll < 0.06 else ["raise", f"shard {s} unreachable"] if roll < 0.1
                      else ["ready", prefix, f"lease-{s}-a", []]]
            for g in range(n_groups):
                roll = rng.random()
                here = positions[g][s]
                if roll < 0.05:
                    script.append(["loading"])
                elif roll < 0.1:
                    script.append(["ready", len(here) + 1, f"lease-{s}-g{g}", here])
                elif roll < 0.14:
                    script.append(["raise", f"shard {s} dropped"])
                else:
                    script.append(["ready", len(here), f"lease-{s}-g{g}" if rng.random() > 0.05 else "", here])
            roll = rng.random()
            script.append(["loading"] if roll < 0.1 else ["ready", max(0, reconciled - 1), f"lease-{s}-x", []] if roll < 0.2
                          else ["ready", reconciled, f"lease-{s}-x", []])
            scripts.append(script)
        failing = [f"lease-{s}-a" for s in range(n_shards) if rng.random() < 0.08]
        out.append(["hybrid", n_hashes, scripts, failing, list(range(1, n_groups + 1))])
    return out


def run_hybrid(make_client, ready_cls, loading_cls, seed=78):
    results = []
    for kind, n_hashes, scripts, failing, group_ids in hybrid_scenarios(random.Random(seed)):
        log = []
        shards = tuple(ScriptedShard(i, [list(step) for step in sc], log, ready_cls, loading_cls, failing)
                       for i, sc in enumerate(scripts))
        client = make_client(shards, group_ids)
        hashes = [b"h%d" % i for i in range(n_hashes)]
        outcome = _outcome(lambda: client.hybrid("inst", hashes, "req", False))
        results.append({"kind": kind, "n_hashes": n_hashes, "scripts": scripts, "groups": group_ids, "outcome": outcome,
                        "log": log})
    return results


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
