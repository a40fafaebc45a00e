"""Scheduler-side half of the connector: decides, per scheduling step, which blocks a worker
loads from the host pool and which it saves to it.

Mirrors the reference's ``SchedulerConnector`` (python/pegaflow/connector/scheduler.py) and
``TpShardQueryClient`` (python/pegaflow/connector/tp_shards.py): prefix lookup with query leases,
the identity check that protects a lookup against a request that moved on while a slower tier
was loading, load intents after block allocation, incremental save intents as blocks fill up, and
the hold on a finished request's blocks until its saves have been sent.  With a cache-group
layout that has recurrent-state groups (hybrid attention + Mamba models) the reference's hybrid
rules apply: a hit ends at a checkpoint every recurrent group holds on every shard, the recurrent
groups load only that checkpoint's state block, blocks are saved from vLLM's block pool by hash,
and the last state block is saved when the request finishes.  Not mirrored: the prefill/decode
tail-block extension.  (The vLLM plug-in and the worker-side mirror in this package serve one
attention or MLA group; they do not consume the recurrent holds.)

Everything here is host bookkeeping over block ids, hashes and leases; no KV bytes are touched.
The objects it reads are vLLM's (``Request.request_id/.block_hashes/.num_tokens``,
``KVCacheBlocks.get_block_ids()/.blocks``, ``SchedulerOutput.scheduled_new_reqs/
.scheduled_cached_reqs/.num_scheduled_tokens/.preempted_req_ids``) and are duck-typed.
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Dict, List, Optional, Sequence, Tuple

from .config import CacheGroupLayout, reconcile_hybrid_hit
from .connector import QueryLoading, QueryReady


@dataclass(frozen=True)
class RecurrentLoadHold:
    """Pinned recurrent-state checkpoints of one hybrid load (common.py:233-249): `leases[g][shard]`
    is the membership lease over recurrent group g's hit blocks on that shard, `hit_positions[g][shard]`
    their positions in the query (lease order), `checkpoint` the position the load resumes from —
    the state stored there covers every token up to the end of that block."""
    leases: Tuple[Tuple[bytes, ...], ...]
    hit_positions: Tuple[Tuple[Tuple[int, ...], ...], ...]
    checkpoint: int


@dataclass(frozen=True)
class LoadIntent:
    """common.py:220-231."""
    block_ids_by_group: Tuple[Tuple[Optional[int], ...], ...]
    leases: Tuple[bytes, ...]
    num_tokens: int
    recurrent_hold: Optional[RecurrentLoadHold] = None


@dataclass(frozen=True)
class SaveIntent:
    """common.py:288-293."""
    block_ids_by_group: Tuple[Tuple[int, ...], ...]
    block_hashes: Tuple[bytes, ...]


class PegaConnectorMetadata:
    """What the scheduler hands the workers for one step (common.py:440-461)."""

    def __init__(self, load_intents=None, save_intents=None, ready_save_intents=None, preempted_req_ids=None):
        self.load_intents: Dict[str, LoadIntent] = load_intents or {}
        self.save_intents: Dict[str, SaveIntent] = save_intents or {}
        self.ready_save_intents: Dict[str, SaveIntent] = ready_save_intents or {}
        self.preempted_req_ids: set = preempted_req_ids or set()

    def __repr__(self):
        return (f"PegaConnectorMetadata(loads={len(self.load_intents)}, saves={len(self.save_intents)}, "
                f"ready_saves={len(self.ready_save_intents)})")


@dataclass
class _Probe:
    """One prefix lookup: what was asked (the request's position and remaining hashes at that
    moment) and, once the backend answered Ready, how many blocks it holds under which leases."""
    computed_blocks: int
    hashes: Tuple[bytes, ...]
    hit_blocks: Optional[int] = None      # None: the backend is still loading
    leases: Tuple[bytes, ...] = ()
    hold: Optional[RecurrentLoadHold] = None     # hybrid models: the pinned recurrent checkpoints
    usable: frozenset = frozenset()              # hybrid models: every position the hit may end at

    def same_query(self, computed_blocks: int, hashes: Tuple[bytes, ...]) -> bool:
        return self.computed_blocks == computed_blocks and self.hashes == hashes


@dataclass
class _Tracked:
    """Save-side state of a request from its first allocation to its cleanup."""
    request: object
    hashes: Tuple[bytes, ...]
    first_local_block: int                 # blocks before this index came from the host pool
    next_to_store: int
    block_ids: List[List[int]] = field(default_factory=list)     # per cache group, in request order
    scheduled_tokens: int = 0


def require_single_attention_group(kv_cache_config) -> None:
    """Accept what this scheduler connector can serve and refuse the rest loudly: one KV-cache
    group of full-attention or MLA layers (or a uniformly typed group of MLA layers), the
    single-group cases of the reference's `CacheGroupLayout.from_config` (common.py:305-356).
    Hybrid configurations (attention + recurrent-state groups) need the reference's reconcile
    logic, which is not mirrored.  Specs are matched by class name so that vLLM need not be
    importable where this runs."""
    groups = tuple(getattr(kv_cache_config, "kv_cache_groups", ()) or ())
    if not groups:
        return
    if len(groups) > 1:
        raise RuntimeError(f"this connector supports a single KV cache group, the model has {len(groups)} "
                           "(hybrid attention + recurrent-state caches are not supported)")
    def kinds(obj):
        return {c.__name__ for c in type(obj).__mro__}

    spec = groups[0].kv_cache_spec
    kind = type(spec).__name__
    if kinds(spec) & {"FullAttentionSpec", "MLAAttentionSpec"}:
        return
    if kind == "UniformTypeKVCacheSpecs":
        inner = list((getattr(spec, "kv_cache_specs", None) or {}).values())
        if inner and all("MLAAttentionSpec" in kinds(x) for x in inner):
            return
    raise RuntimeError("this connector supports a single cache group only for FullAttention, MLA, or uniformly "
                       f"grouped MLA layers (got {kind})")


@dataclass(frozen=True)
class HybridHit:
    """Outcome of `ShardQuery.query_hybrid`: the attention prefix leases (one per shard) and, for a
    hit, the pinned recurrent checkpoints — `recurrent_leases[g][shard]` over the blocks at
    `recurrent_positions[g][shard]` — with the chosen checkpoint position and every position the
    hit may legally end at (common.py:233-249, tp_shards.py:9-19)."""
    num_hit_blocks: int
    leases: Tuple[bytes, ...]
    recurrent_leases: Tuple[Tuple[bytes, ...], ...] = ()
    recurrent_positions: Tuple[Tuple[Tuple[int, ...], ...], ...] = ()
    checkpoint: Optional[int] = None
    usable_positions: Tuple[int, ...] = ()


class ShardQuery:
    """Prefix query across node-local TP shards (tp_shards.py:23-97): the usable hit is the prefix
    every shard holds; shards that answered with more are re-leased for exactly that prefix."""

    def __init__(self, clients: Sequence[object]):
        if not clients:
            raise ValueError("at least one engine client is needed")
        self.clients = tuple(clients)

    def query(self, instance_id: str, hashes: List[bytes], req_id: str, wait_for_full_prefix: bool):
        """(hit blocks, one lease per shard), or None while some shard is still loading."""
        answers: List[QueryReady] = []
        try:
            for index, client in enumerate(self.clients):
                got = client.query_prefetch(instance_id, hashes, req_id=req_id, wait_for_full_prefix=wait_for_full_prefix)
                if _is_loading(got):
                    self.release([a.lease for a in answers], req_id)
                    return None
                answers.append(got)      # before the check: a malformed answer's lease is given back too
                self._check(got, len(hashes), index)
        except Exception:
            self.release([a.lease for a in answers], req_id)
            raise
        common = min(a.num_hit_blocks for a in answers)
        leases = [a.lease for a in answers]
        if common == 0:
            self.release(leases, req_id)
            return 0, tuple(b"" for _ in answers)
        try:
            for index, (client, answer) in enumerate(zip(self.clients, answers)):
                if answer.num_hit_blocks == common:
                    continue
                exact = client.query_prefetch(instance_id, hashes[:common], req_id=f"{req_id}:tp-common-{common}",
                                              wait_for_full_prefix=False)
                if _is_loading(exact):
                    raise RuntimeError(f"TP shard {index} could not lease the common {common}-block prefix")
                try:
                    self._check(exact, common, index)
                    if exact.num_hit_blocks != common:
                        raise RuntimeError(f"TP shard {index} could not lease the common {common}-block prefix")
                except Exception:
                    self._release_one(client, exact.lease)
                    raise
                longer, leases[index] = leases[index], exact.lease
                self._release_one(client, longer)
        except Exception:
            self.release(leases, req_id)
            raise
        return common, tuple(leases)

    def query_group_membership(self, instance_id: str, hashes: List[bytes], req_id: str, group_id: int):
        """Which of `hashes` one hybrid storage group holds, per shard (tp_shards.py:93-141): a list of
        (hit positions, lease over exactly those blocks, in that order).  Membership is answered from
        memory only, so a shard that says Loading is an error; whatever goes wrong, the leases of the
        shards that had already answered are given back."""
        answers: List[Tuple[Tuple[int, ...], bytes]] = []
        try:
            for index, client in enumerate(self.clients):
                got = client.query_prefetch(instance_id, hashes, req_id=req_id, group_id=group_id)
                if isinstance(got, QueryLoading) or type(got).__name__ == "QueryLoading":
                    raise RuntimeError(f"TP shard {index} membership query for group {group_id} returned Loading; "
                                       "membership queries are local-only")
                if not hasattr(got, "num_hit_blocks"):
                    raise TypeError(f"query_prefetch returned unexpected outcome {type(got)!r}")
                positions = tuple(got.hit_positions)
                if len(positions) != got.num_hit_blocks:
                    raise RuntimeError(f"TP shard {index} reported {got.num_hit_blocks} hits but returned "
                                       f"{len(positions)} positions")
                if any(p >= len(hashes) for p in positions):
                    raise RuntimeError(f"TP shard {index} returned hit positions outside a {len(hashes)}-hash query")
                if positions and not got.lease:
                    raise RuntimeError(f"TP shard {index} returned {len(positions)} hits without a lease")
                answers.append((positions, got.lease))
        except Exception:
            self.release([lease for _, lease in answers], req_id)
            raise
        return answers

    def query_hybrid(self, instance_id: str, hashes: List[bytes], req_id: str, wait_for_full_prefix: bool,
                     recurrent_group_ids: Sequence[int]):
        """Prefix query for a hybrid (attention + recurrent state) model (scheduler.py:927-1075): the
        attention prefix only counts as far as every recurrent storage group has a state checkpoint
        on every shard.  Returns None while a shard is loading, else a `HybridHit`; a hit of 0 blocks
        means every lease taken on the way has been given back."""
        answer = self.query(instance_id, hashes, req_id, wait_for_full_prefix)
        if answer is None:
            return None
        hit, leases = answer
        if hit == 0:
            return HybridHit(0, leases)
        members: List[List[Tuple[Tuple[int, ...], bytes]]] = []

        def release_members():
            for gid, group in zip(recurrent_group_ids, members):
                self.release([lease for _, lease in group], f"{req_id}:g{gid}")

        try:
            for gid in recurrent_group_ids:
                members.append(self.query_group_membership(instance_id, hashes, f"{req_id}:g{gid}", gid))
            blocks, checkpoint, usable = reconcile_hybrid_hit(
                hit, tuple(tuple(positions for positions, _ in group) for group in members))
        except Exception:
            self.release(leases, req_id)
            release_members()
            raise
        nothing = HybridHit(0, tuple(b"" for _ in leases))
        if blocks == 0 or checkpoint is None:
            self.release(leases, req_id)
            release_members()
            return nothing
        if blocks < hit:
            # the usable prefix is shorter than the leased one: lease exactly what will be loaded
            exact = self.query(instance_id, hashes[:blocks], f"{req_id}:hma-exact-{blocks}", False)
            self.release(leases, req_id)
            if exact is None or exact[0] != blocks:
                if exact is not None:
                    self.release(exact[1], req_id)
                release_members()
                return nothing
            leases = exact[1]
        return HybridHit(blocks, leases,
                         tuple(tuple(lease for _, lease in group) for group in members),
                         tuple(tuple(positions for positions, _ in group) for group in members),
                         checkpoint, tuple(sorted(usable)))

    def release(self, leases: Sequence[bytes], req_id: str = "") -> bool:
        ok = True
        for client, lease in zip(self.clients, leases):
            ok = self._release_one(client, lease) and ok
        return ok

    @staticmethod
    def _release_one(client, lease: bytes) -> bool:
        if not lease:
            return True
        try:
            client.release(lease)
        except Exception:
            return False
        return True

    @staticmethod
    def _check(answer, asked: int, index: int):
        if answer.num_hit_blocks > asked:
            raise RuntimeError(f"TP shard {index} reported {answer.num_hit_blocks} hits for a {asked}-block query")
        if answer.num_hit_blocks and not answer.lease:
            raise RuntimeError(f"TP shard {index} returned {answer.num_hit_blocks} hits without a lease")


def _is_loading(answer) -> bool:
    # A client may answer with its own Loading type (the reference's native client does): anything
    # that carries no hit count is "still loading".
    return isinstance(answer, QueryLoading) or not hasattr(answer, "num_hit_blocks")


class SchedulerConnector:
    def __init__(self, clients: Sequence[object], *, instance_id: str, block_size: int, read_enabled: bool = True,
                 wait_for_full_prefix: bool = False, cache_groups: Optional[CacheGroupLayout] = None):
        self.instance_id, self.block_size = instance_id, block_size
        self.read_enabled, self.wait_for_full_prefix = read_enabled, wait_for_full_prefix
        self._shards = ShardQuery(clients)
        # one attention (or MLA) group unless told otherwise; a layout with recurrent-state groups turns
        # on the hybrid rules (lookups gated on a common checkpoint, saves taken from the local cache)
        self._groups = cache_groups or CacheGroupLayout(((),), 0, False, frozenset(), frozenset())
        self._recurrent_storage_ids = tuple(self._groups.storage_group_ids[i]
                                            for i in sorted(self._groups.recurrent_group_indices))
        self._local_cached_block = None
        self._probes: Dict[str, _Probe] = {}
        self._matched_blocks: Dict[str, int] = {}      # local prefix + blocks to be loaded, per request
        self._tracked: Dict[str, _Tracked] = {}
        self._loads: Dict[str, LoadIntent] = {}
        self._deferred_saves: Dict[str, SaveIntent] = {}
        self._unsent: set = set()                      # requests with saves the workers have not reported sent
        self._held: set = set()                        # finished requests whose blocks wait for those saves

    def bind_gpu_block_pool(self, gpu_block_pool) -> None:
        """scheduler.py:197-208.  Hybrid saves name blocks by hash through vLLM's block pool; and with
        more than one group vLLM's own prefix cache could expose a loaded attention group before the
        recurrent group has a usable state, so local prefix hits are switched off there."""
        self._local_cached_block = gpu_block_pool.get_cached_block
        if self._groups.group_count > 1:
            gpu_block_pool.get_cached_block = lambda *_a, **_k: None

    def _lookup(self, hashes: List[bytes], req_id: str):
        """None while loading, else (hit blocks, prefix leases, recurrent hold or None, usable positions)."""
        if self._groups.has_recurrent_state:
            got = self._shards.query_hybrid(self.instance_id, hashes, req_id, self.wait_for_full_prefix,
                                            self._recurrent_storage_ids)
            if got is None:
                return None
            hold = None
            if got.checkpoint is not None:
                hold = RecurrentLoadHold(got.recurrent_leases, got.recurrent_positions, got.checkpoint)
            return got.num_hit_blocks, got.leases, hold, frozenset(got.usable_positions)
        got = self._shards.query(self.instance_id, hashes, req_id, self.wait_for_full_prefix)
        return None if got is None else (got[0], got[1], None, frozenset())

    def _release_hold(self, hold: Optional[RecurrentLoadHold], req_id: str) -> bool:
        ok = True
        for index, leases in enumerate(hold.leases if hold is not None else ()):
            ok = self._shards.release(leases, f"{req_id}:g{index}") and ok
        return ok

    # ------------------------------------------------------------------ lookup (scheduler.py:210-407)
    def get_num_new_matched_tokens(self, request, num_computed_tokens: int) -> Tuple[Optional[int], bool]:
        """(tokens the host pool can supply beyond the local prefix, load asynchronously?) or
        (None, False) while a slower tier is still fetching and the scheduler should ask again."""
        req_id = request.request_id
        if not self.read_enabled:
            return 0, False
        computed = num_computed_tokens // self.block_size
        hashes = tuple(request.block_hashes[computed:])
        if not hashes:
            self._drop_probe(req_id)
            self._matched_blocks[req_id] = computed
            return 0, False

        probe = self._probes.get(req_id)
        if probe is not None and probe.hit_blocks is not None:
            if probe.same_query(computed, hashes):
                return self._answer(req_id, request.num_tokens, probe)
            self._drop_probe(req_id)      # a Ready for a query the request has left behind: give the lease back
            probe = None

        # A lookup that is loading is known to the backend by request id: keep polling with the
        # hashes it was started with, and compare the answer with today's position afterwards.
        moved_on = probe is not None and not probe.same_query(computed, hashes)
        answer = self._lookup(list(probe.hashes if moved_on else hashes), req_id)
        if answer is None:
            if probe is None:
                self._probes[req_id] = _Probe(computed, hashes)
            return None, False
        hit_blocks, leases, hold, usable = answer
        if moved_on:
            self._shards.release(leases, req_id)
            self._release_hold(hold, req_id)
            self._probes.pop(req_id, None)
            return None, False
        if probe is None:
            probe = self._probes[req_id] = _Probe(computed, hashes)
        if hit_blocks > len(probe.hashes):
            raise RuntimeError(f"invariant violated: server returned {hit_blocks} hits for {len(probe.hashes)} hashes")
        probe.hit_blocks, probe.leases, probe.hold, probe.usable = hit_blocks, leases, hold, usable
        return self._answer(req_id, request.num_tokens, probe)

    def _answer(self, req_id: str, num_tokens: int, probe: _Probe) -> Tuple[int, bool]:
        bs = self.block_size
        hit_tokens = probe.hit_blocks * bs
        # one token is always left for the forward pass that produces the first logits
        hit_tokens = min(hit_tokens, max(0, num_tokens - probe.computed_blocks * bs - 1))
        if probe.hold is not None:
            # a recurrent state can only be resumed at the end of its own block: when the clamp cut
            # into the reconciled span, fall back to the last checkpoint before the cut, or give up
            boundary = hit_tokens // bs
            earlier = [p for p in probe.usable if p < boundary]
            if not earlier:
                if self._probes.get(req_id) is probe:
                    self._drop_probe(req_id)
                return 0, False
            checkpoint = max(earlier)
            probe.hit_blocks = checkpoint + 1
            hit_tokens = probe.hit_blocks * bs
            probe.hold = replace(probe.hold, checkpoint=checkpoint)
        self._matched_blocks[req_id] = probe.computed_blocks + (hit_tokens + bs - 1) // bs
        if hit_tokens <= 0:
            self._drop_probe(req_id)
            return 0, False
        return hit_tokens, True

    def pending_lookup_position(self, req_id: str) -> Optional[int]:
        """Locally computed blocks at the time of the request's pending Ready lookup, if any."""
        probe = self._probes.get(req_id)
        return probe.computed_blocks if probe is not None and probe.hit_blocks is not None else None

    # ------------------------------------------------------------------ allocation (scheduler.py:409-497)
    def update_state_after_alloc(self, request, blocks, num_external_tokens: int) -> None:
        req_id = request.request_id
        t = self._tracked.get(req_id)
        if t is None:
            first = self._matched_blocks.get(req_id, 0)
            t = self._tracked[req_id] = _Tracked(request, tuple(request.block_hashes), first, first,
                                                 [[] for _ in range(self._groups.group_count)])
        else:
            t.request, t.hashes = request, tuple(request.block_hashes)
        if num_external_tokens <= 0:
            return
        ids = self._by_group(blocks.get_block_ids()) if blocks else tuple(() for _ in range(self._groups.group_count))
        hashed = blocks.blocks[self._groups.hash_group_index] if blocks else ()
        already_computed = sum(b.block_hash is not None for b in hashed)
        n_load = (num_external_tokens + self.block_size - 1) // self.block_size
        if any(len(g) < already_computed + n_load for g in ids):
            self._drop_probe(req_id)
            raise RuntimeError(f"load block mismatch: start={already_computed} count={n_load} "
                               f"available_by_group={[len(g) for g in ids]}")
        destinations = []
        for index, group in enumerate(ids):
            dst = group[already_computed:already_computed + n_load]
            if index in self._groups.recurrent_group_indices and dst:
                dst = (None,) * (len(dst) - 1) + (dst[-1],)     # only the checkpoint's state is loaded
            destinations.append(dst)
        probe = self._probes.get(req_id)
        intent = LoadIntent(tuple(destinations), probe.leases if probe is not None else (), num_external_tokens,
                            probe.hold if probe is not None else None)
        if probe is not None:
            if not probe.same_query(already_computed, tuple(request.block_hashes[already_computed:])):
                self._drop_probe(req_id)
                raise RuntimeError(f"req {req_id} query identity changed before external load")
            if probe.hit_blocks is None:
                raise RuntimeError("query probe is still loading")
            if probe.hit_blocks != n_load:
                self._drop_probe(req_id)
                raise RuntimeError(f"req {req_id} leased block mismatch: leased={probe.hit_blocks} load={n_load}")
        if not intent.leases or any(not lease for lease in intent.leases):
            raise RuntimeError(f"req {req_id} missing query lease for external load")
        self._loads[req_id] = intent
        self._probes.pop(req_id, None)     # the lease now travels with the load intent; the worker consumes it

    # ------------------------------------------------------------------ per step (scheduler.py:499-596)
    def build_connector_meta(self, scheduler_output) -> PegaConnectorMetadata:
        ready_saves, self._deferred_saves = self._deferred_saves, {}
        loads, self._loads = self._loads, {}
        saves: Dict[str, SaveIntent] = {}
        scheduled = scheduler_output.num_scheduled_tokens

        for new in scheduler_output.scheduled_new_reqs:
            t = self._tracked.get(new.req_id)
            assert t is not None, f"req {new.req_id} not initialized in update_state_after_alloc"
            if new.block_ids:
                t.block_ids = [list(g) for g in self._by_group(new.block_ids)]
            self._count_tokens(t, new.num_computed_tokens, scheduled.get(new.req_id, 0))
            intent = self._next_save(t, new.num_computed_tokens)
            if intent:
                saves[new.req_id] = intent

        running = scheduler_output.scheduled_cached_reqs
        for i, req_id in enumerate(running.req_ids):
            t = self._tracked.get(req_id)
            if t is None:
                continue
            t.hashes = tuple(t.request.block_hashes)      # decode completes new blocks: pick up their hashes
            fresh = running.new_block_ids[i]
            if req_id in running.resumed_req_ids:
                t.block_ids = ([list(g) for g in self._by_group(fresh)] if fresh
                               else [[] for _ in range(self._groups.group_count)])
            elif fresh:
                for have, more in zip(t.block_ids, self._by_group(fresh)):
                    have.extend(more)
            self._count_tokens(t, running.num_computed_tokens[i], scheduled.get(req_id, 0))
            intent = self._next_save(t, running.num_computed_tokens[i])
            if intent:
                saves[req_id] = intent

        self._unsent.update(saves)
        return PegaConnectorMetadata(loads, saves, ready_saves, set(scheduler_output.preempted_req_ids or ()))

    def _count_tokens(self, t: _Tracked, computed_before: int, now: int):
        if self.read_enabled:
            t.scheduled_tokens += now
        else:
            t.scheduled_tokens = max(t.scheduled_tokens, computed_before + now)

    def _next_save(self, t: _Tracked, computed_before_step: int) -> Optional[SaveIntent]:
        """Blocks that became full since the last step (scheduler.py:700-770): block ids and hashes
        are both in request order, and the prefix that was loaded from the pool is never re-saved.
        Hybrid models save only what was complete before this step and take the block ids from
        vLLM's block pool by hash (every group's block of a hash, or nothing yet)."""
        hybrid = self._groups.has_recurrent_state
        if hybrid:
            end = min(len(t.hashes), computed_before_step // self.block_size)
        else:
            full_local = min(min((len(g) for g in t.block_ids), default=0), t.scheduled_tokens // self.block_size)
            end = min(len(t.hashes), t.first_local_block + full_local)
        if end <= t.next_to_store:
            return None
        start = t.next_to_store
        hashes = t.hashes[start:end]
        if hybrid:
            ids = self._local_cached_ids(hashes)
            if ids is None:
                return None
        else:
            ids = tuple(tuple(g[start:end]) for g in t.block_ids)
        t.next_to_store = end
        return SaveIntent(ids, hashes)

    def _local_cached_ids(self, hashes: Sequence[bytes]):
        """scheduler.py:774-789."""
        if self._local_cached_block is None:
            raise RuntimeError("HMA block pool was not bound before building save metadata")
        group_ids = list(range(self._groups.group_count))
        out: List[List[int]] = [[] for _ in group_ids]
        for h in hashes:
            cached = self._local_cached_block(h, group_ids)
            if cached is None:
                return None
            for ids, block in zip(out, cached):
                ids.append(block.block_id)
        return tuple(tuple(ids) for ids in out)

    def _final_hybrid_save(self, t: _Tracked, block_ids, written: int) -> Optional[SaveIntent]:
        """What a finished hybrid request still has to save (scheduler.py:791-837): the attention
        blocks not saved yet, and for every recurrent group only the state block that follows the
        last full block — the null block stands in for the positions before it."""
        start = t.next_to_store
        end = min(len(t.hashes), written // self.block_size)
        if end <= start:
            return None
        groups = self._by_group(block_ids)
        recurrent = self._groups.recurrent_group_indices
        available = tuple(len(g) for g in groups)
        required = tuple(end + 1 if i in recurrent else end for i in range(self._groups.group_count))
        if any(have < need for have, need in zip(available, required)):
            raise RuntimeError(f"req {t.request.request_id} final HMA block table is shorter than its hash prefix: "
                               f"saveable={end} available_by_group={available} required_by_group={required}")
        ids = tuple((0,) * (end - start - 1) + (g[end],) if i in recurrent else g[start:end]
                    for i, g in enumerate(groups))
        t.next_to_store = end
        return SaveIntent(ids, t.hashes[start:end])

    # ------------------------------------------------------------------ completion (scheduler.py:874-925)
    def update_connector_output(self, connector_output) -> None:
        for req_id in connector_output.finished_sending or []:
            self._unsent.discard(req_id)
            if req_id in self._held and req_id not in self._deferred_saves:
                self._forget(req_id)
                self._held.discard(req_id)

    def request_finished(self, request, block_ids) -> Tuple[bool, Optional[dict]]:
        """True: the caller must keep the request's blocks until its saves are reported sent."""
        req_id = request.request_id
        t = self._tracked.get(req_id)
        if self._groups.has_recurrent_state and t is not None:
            t.hashes = tuple(request.block_hashes)
            final = self._final_hybrid_save(t, block_ids, request.num_computed_tokens)
            if final is not None:
                self._deferred_saves[req_id] = final
                self._unsent.add(req_id)
        if req_id in self._unsent:
            self._held.add(req_id)
            return True, None
        self._forget(req_id)
        return False, None

    def shutdown(self) -> None:
        for req_id in list(self._probes):
            self._drop_probe(req_id)

    # ------------------------------------------------------------------ helpers
    def _forget(self, req_id: str):
        self._drop_probe(req_id)
        self._tracked.pop(req_id, None)
        self._matched_blocks.pop(req_id, None)
        self._deferred_saves.pop(req_id, None)
        self._unsent.discard(req_id)

    def _drop_probe(self, req_id: str) -> bool:
        probe = self._probes.pop(req_id, None)
        if probe is None:
            return True
        ok = self._shards.release(probe.leases, req_id) if any(probe.leases) else True
        return self._release_hold(probe.hold, req_id) and ok

    def _by_group(self, block_ids) -> Tuple[Tuple[int, ...], ...]:
        groups = tuple(tuple(g) for g in block_ids)
        if len(groups) != self._groups.group_count:
            raise RuntimeError(f"KV cache group count mismatch: expected={self._groups.group_count} actual={len(groups)}")
        if any(b < 0 for g in groups for b in g):
            raise RuntimeError("KV cache block IDs must be non-negative")
        return groups
