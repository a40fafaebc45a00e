"""CPU model of the reference engine's save/load path, built on the C oracle.

TEST INFRASTRUCTURE ONLY (see ``pf_oracle.py``).  "GPU memory" here is a numpy byte buffer
whose address is registered as ``data_ptr``; the "pinned pool" is another numpy buffer.  The
model follows the reference's control flow closely enough that the same call sequence can be
replayed against the CUDA engine and compared byte for byte:

* registration and topology sealing  — pegaflow-core/src/lib.rs:302-440, instance.rs:500-672,757-825
* save phases 0-4                    — pegaflow-core/src/offload.rs:182-282,293-659,
                                       storage/write_path.rs:119-254
* prefix query / leases              — storage/read_cache.rs:64-80, lease.rs:83-153
* load target mapping                — pegaflow-core/src/lib.rs:715-895

Absolute pool offsets are NOT part of the contract (the reference takes them from a third-party
allocator); parity is defined on GPU bytes after a load and on each stored block's host image.
"""

from __future__ import annotations

import os
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from . import pf_oracle as po


class EngineError(Exception):
    """Mirror of ``EngineError`` (pegaflow-core/src/lib.rs:72-103); ``str()`` is its Display."""

    FORMATS = {
        "InstanceMissing": "instance {0} not found",
        "WorkerMissing": "device {1} not found in instance {0}",
        "InvalidArgument": "invalid argument: {0}",
        "CudaInit": "failed to initialize CUDA: {0}",
        "Storage": "storage error: {0}",
        "Poisoned": "internal lock poisoned: {0}",
        "TopologyMismatch": "topology mismatch: {0}",
    }

    def __init__(self, kind: str, *args):
        self.kind = kind
        self.args_ = args
        super().__init__(self.FORMATS[kind].format(*args))


def _invalid(msg):
    return EngineError("InvalidArgument", msg)


class _Pool:
    """First-fit allocator over a numpy buffer; sizes rounded up to the reference's unit."""

    def __init__(self, nbytes: int, unit_hint: Optional[int] = None):
        self.unit = po.pool_unit_size(nbytes, unit_hint)
        self.capacity = nbytes // self.unit * self.unit
        self.buf = np.zeros(max(self.capacity, 1), dtype=np.uint8)
        self.base = self.buf.ctypes.data
        self.free: List[Tuple[int, int]] = [(0, self.capacity)]
        self.next_id = 1

    def allocate(self, size: int):
        need = (size + self.unit - 1) // self.unit * self.unit
        for i, (off, ln) in enumerate(self.free):
            if ln >= need:
                if ln == need:
                    self.free.pop(i)
                else:
                    self.free[i] = (off + need, ln - need)
                aid = self.next_id
                self.next_id += 1
                return _Alloc(self, off, need, aid)
        return None

    def release(self, off, ln):
        self.free.append((off, ln))
        self.free.sort()
        merged = []
        for o, l in self.free:
            if merged and merged[-1][0] + merged[-1][1] == o:
                merged[-1] = (merged[-1][0], merged[-1][1] + l)
            else:
                merged.append((o, l))
        self.free = merged


@dataclass
class _Alloc:
    pool: _Pool
    offset: int
    size: int
    ident: int

    @property
    def host(self):
        return self.pool.base + self.offset


@dataclass
class _Segment:
    alloc: _Alloc
    offset_in_alloc: int
    size: int

    @property
    def host(self):
        return self.alloc.host + self.offset_in_alloc

    def bytes(self) -> bytes:
        o = self.alloc.offset + self.offset_in_alloc
        return self.alloc.pool.buf[o:o + self.size].tobytes()


@dataclass
class _RawBlock:
    segments: List[_Segment]


@dataclass
class SealedBlock:
    slots: List[Optional[_RawBlock]]

    def get_slot(self, slot_id):
        return self.slots[slot_id] if slot_id < len(self.slots) else None


@dataclass
class _Gpu:
    device_id: int
    tp_rank: int
    pp_rank: int
    layouts: Dict[str, po.KVCacheLayout]
    groups: Dict[str, int]


@dataclass
class _Topology:
    name_to_id: Dict[str, int]
    tp_size: int
    layer_group: List[int]
    group_layer_count: List[int]
    layer_group_rank: List[int]
    page: Optional[dict]

    def layer_id(self, name):
        if name not in self.name_to_id:
            raise _invalid(f"layer {name} is not registered")
        return self.name_to_id[name]

    @property
    def num_layers(self):
        return len(self.name_to_id)

    def total_slots(self):
        return len(self.page["shard_page_sizes"]) if self.page else self.num_layers * self.tp_size

    def group_total_slots(self, g):
        if g >= len(self.group_layer_count):
            raise _invalid(f"storage group {g} out of range ({len(self.group_layer_count)} groups)")
        return len(self.page["shard_page_sizes"]) if self.page else self.group_layer_count[g] * self.tp_size

    def slot_index(self, layer_id, tp_rank):
        if layer_id >= self.num_layers:
            raise _invalid(f"layer_id {layer_id} out of range ({self.num_layers} layers)")
        if tp_rank >= self.tp_size:
            raise _invalid(f"tp_rank {tp_rank} out of range (tp_size {self.tp_size})")
        if self.page:
            return self.page["layer_shard"][layer_id]
        return self.layer_group_rank[layer_id] * self.tp_size + tp_rank

    def page_placement(self, layer_id):
        if not self.page:
            return None
        return self.page["layer_offsets"][layer_id], self.page["layer_bytes"][layer_id]


@dataclass
class _Instance:
    ident: str
    namespace: str
    tp_size: int
    world_size: int
    page_first: bool
    gpus: Dict[int, _Gpu] = field(default_factory=dict)
    topology: Optional[_Topology] = None


class OracleEngine:
    """The reference engine's observable behaviour on CPU memory."""

    def __init__(self, pool_bytes: int, *, ssd_alignment: int = 0, blockwise_alloc: bool = False,
                 unit_hint: Optional[int] = None):
        self.pool = _Pool(pool_bytes, unit_hint)
        self.ssd_alignment = ssd_alignment
        self.blockwise = blockwise_alloc
        self.instances: Dict[str, _Instance] = {}
        self.read_cache: Dict[Tuple[str, bytes], SealedBlock] = {}
        self.inflight: Dict[Tuple[str, bytes], Tuple[int, Dict[int, _RawBlock]]] = {}
        self.inflight_born: Dict[Tuple[str, bytes], float] = {}
        self.leases: Dict[bytes, list] = {}

    # -- registration: lib.rs:302-440 ----------------------------------------------------------
    def register_context_layer_batch_strided(self, instance_id, namespace, device_id, tp_rank, pp_rank, tp_size,
                                             world_size, layer_names, data_ptrs, size_bytes, num_blocks,
                                             bytes_per_block, kv_stride_bytes, segments, block_stride_bytes=None,
                                             layer_group_ids=None, transfer_mode="direct", page_first=False):
        n = len(layer_names)
        lens = [len(x) for x in (data_ptrs, size_bytes, num_blocks, bytes_per_block, kv_stride_bytes, segments)]
        if any(l != n for l in lens):
            raise _invalid(
                f"registration metadata length mismatch: layer_names={n}, data_ptrs={lens[0]}, size_bytes={lens[1]}, "
                f"num_blocks={lens[2]}, bytes_per_block={lens[3]}, kv_stride_bytes={lens[4]}, segments={lens[5]}")
        if block_stride_bytes is not None and len(block_stride_bytes) != n:
            raise _invalid(f"registration metadata length mismatch: layer_names={n}, "
                           f"block_stride_bytes={len(block_stride_bytes)}")
        if layer_group_ids is not None and len(layer_group_ids) != n:
            raise _invalid(f"registration metadata length mismatch: layer_names={n}, "
                           f"layer_group_ids={len(layer_group_ids)}")
        layouts: Dict[str, po.KVCacheLayout] = {}
        for i, name in enumerate(layer_names):
            try:
                lay = po.KVCacheLayout(data_ptrs[i], size_bytes[i], num_blocks[i], bytes_per_block[i],
                                       kv_stride_bytes[i], segments[i])
                if block_stride_bytes is not None:
                    lay.with_block_stride(block_stride_bytes[i])
            except po.OracleError as e:
                raise _invalid(f"layer {name}: {e}") from None
            if self.ssd_alignment:
                lay.with_ssd_padding(self.ssd_alignment)
            if name in layouts:
                raise _invalid(f"duplicate layer name in registration batch: {name}")
            layouts[name] = lay
        groups = dict(zip(layer_names, layer_group_ids)) if layer_group_ids is not None else {}

        inst = self.instances.get(instance_id)
        if inst is not None:
            if (inst.tp_size, inst.world_size, inst.page_first) != (tp_size, world_size, bool(page_first)):
                b = lambda v: "true" if v else "false"
                raise EngineError(
                    "TopologyMismatch",
                    f"instance {instance_id} exists with tp={inst.tp_size}, world={inst.world_size}, "
                    f"page_first={b(inst.page_first)}; requested tp={tp_size}, world={world_size}, "
                    f"page_first={b(page_first)}")
        else:
            if tp_size == 0 or world_size == 0:
                raise _invalid("tp_size and world_size must be > 0")
            inst = _Instance(instance_id, namespace, tp_size, world_size, bool(page_first))
            self.instances[instance_id] = inst

        # instance.rs:757-825
        if tp_rank >= inst.tp_size:
            raise _invalid(f"tp_rank {tp_rank} out of range (tp_size {inst.tp_size})")
        if not layouts:
            raise _invalid(f"device {device_id} registered no KV cache layers")
        if device_id in inst.gpus:
            raise _invalid(f"GPU context for device {device_id} already exists")
        if inst.topology is not None:
            raise _invalid(f"instance {inst.ident} is already fully registered ({inst.world_size} workers); "
                           f"device {device_id} cannot join")
        if device_id < 0:
            raise _invalid(f"device_id {device_id} must be >= 0")
        gpu = _Gpu(device_id, tp_rank, pp_rank, layouts, groups)
        if len(inst.gpus) + 1 == inst.world_size:
            inst.topology = self._seal(inst, list(inst.gpus.values()) + [gpu])
        inst.gpus[device_id] = gpu

    def _seal(self, inst: _Instance, gpus: List[_Gpu]) -> _Topology:
        """instance.rs:500-672."""
        geometry: Dict[str, tuple] = {}
        for g in gpus:
            for name, lay in g.layouts.items():
                geo = (lay.segment_bytes, lay.is_split, lay.padded_block_bytes)
                if name in geometry and geometry[name] != geo:
                    raise _invalid(f"layer {name} registered with inconsistent geometry")
                geometry[name] = geo
        names = sorted(geometry.keys(), key=lambda s: s.encode())  # byte-wise order, instance.rs:544-550
        name_to_id = {nm: i for i, nm in enumerate(names)}
        group_by_name: Dict[str, int] = {}
        for g in gpus:
            for name in g.layouts:
                grp = g.groups.get(name, 0)
                if name in group_by_name and group_by_name[name] != grp:
                    raise _invalid(f"layer {name} registered in storage group {group_by_name[name]} on one device "
                                   f"but group {grp} on device {g.device_id}")
                group_by_name[name] = grp
        num_groups = 1 + max(group_by_name.values(), default=0)
        if len(set(group_by_name.values())) != num_groups:
            raise _invalid(f"storage groups must be dense 0..{num_groups}: an unregistered group would never "
                           "seal its blocks")
        layer_group = [0] * len(names)
        layer_group_rank = [0] * len(names)
        group_layer_count = [0] * num_groups
        for nm in names:
            lid = name_to_id[nm]
            grp = group_by_name[nm]
            layer_group[lid] = grp
            layer_group_rank[lid] = group_layer_count[grp]
            group_layer_count[grp] += 1
        if inst.page_first and num_groups > 1:
            raise _invalid(f"page-first storage does not support multiple storage groups ({num_groups} registered)")
        owners: List[Optional[Tuple[int, int]]] = [None] * (len(names) * inst.tp_size)
        for g in gpus:
            for name in g.layouts:
                grid = name_to_id[name] * inst.tp_size + g.tp_rank
                if owners[grid] is None:
                    owners[grid] = (g.device_id, g.pp_rank)
                elif owners[grid][1] != g.pp_rank:
                    raise _invalid(f"layer {name} claimed by different pipeline stages")
        for idx, o in enumerate(owners):
            if o is None:
                raise _invalid(f"instance {inst.ident} has incomplete KV registration: layer "
                               f"{names[idx // inst.tp_size]} has no owner for tp_rank {idx % inst.tp_size} after "
                               f"all {inst.world_size} workers registered")
        page = None
        if inst.page_first:
            sets = [[name_to_id[nm] for nm in g.layouts] for g in gpus]
            padded = [geometry[nm][2] for nm in names]
            try:
                page = po.build_page_layout(sets, len(names), padded)
            except po.OracleError as e:
                raise _invalid(str(e)) from None
        return _Topology(name_to_id, inst.tp_size, layer_group, group_layer_count, layer_group_rank, page)

    def unregister_instance(self, instance_id):
        if self.instances.pop(instance_id, None) is None:
            raise EngineError("InstanceMissing", instance_id)
        self.leases = {k: v for k, v in self.leases.items() if v[0] != instance_id}

    # lib.rs:459-489
    def unregister_all_instances(self) -> List[str]:
        ids = sorted(self.instances)
        self.instances.clear()
        self.leases.clear()
        return ids

    def list_instance_ids(self) -> List[str]:
        return sorted(self.instances)

    def instance_namespace(self, instance_id) -> str:
        return self._instance(instance_id).namespace

    def cleanup_memory_cache(self) -> Dict[str, int]:
        """storage/mod.rs:395-445: every resident block leaves the cache; the ones a lease still holds are counted.
        `reclaimed_bytes` depends on how the pool's allocations were grouped, which the model does not track."""
        held = {id(b) for ent in self.leases.values() for b in ent[1]}
        removed = list(self.read_cache.values())
        self.read_cache.clear()
        footprint = sum(seg.size for b in removed for raw in b.slots if raw is not None for seg in raw.segments)
        return {"evicted_blocks": len(removed), "evicted_bytes": footprint,
                "still_referenced_blocks": sum(1 for b in removed if id(b) in held)}

    def gc_stale_inflight(self, max_age_seconds: float) -> int:
        """lib.rs:938-948: drop the blocks that have waited longer than `max_age_seconds` for slots that never came."""
        if not max_age_seconds >= 0:
            raise _invalid("max_age_seconds must be >= 0")
        now = time.monotonic()
        stale = [k for k, born in self.inflight_born.items() if now - born > max_age_seconds]
        for k in stale:
            self.inflight.pop(k, None)
            del self.inflight_born[k]
        return len(stale)

    def _instance(self, instance_id) -> _Instance:
        if instance_id not in self.instances:
            raise EngineError("InstanceMissing", instance_id)
        return self.instances[instance_id]

    def _sealed(self, inst: _Instance) -> _Topology:
        if inst.topology is None:
            raise _invalid(f"instance {inst.ident} registration incomplete: {len(inst.gpus)}/{inst.world_size} "
                           "workers registered")
        return inst.topology

    def _alloc(self, size, what) -> _Alloc:
        a = self.pool.allocate(size)
        if a is None:
            raise EngineError("Storage", f"pinned pool exhausted while allocating {what}")
        return a

    # -- save: offload.rs:293-659 ---------------------------------------------------------------
    def batch_save(self, instance_id, tp_rank, pp_rank, device_id, saves: Sequence[Tuple[str, Sequence[int],
                                                                                           Sequence[bytes]]]):
        inst = self._instance(instance_id)
        topo = self._sealed(inst)
        gpu = inst.gpus.get(device_id)
        if gpu is None:
            raise EngineError("WorkerMissing", instance_id, device_id)
        if gpu.tp_rank != tp_rank or gpu.pp_rank != pp_rank:
            raise _invalid(f"device_id {device_id} is registered for tp_rank {gpu.tp_rank}, pp_rank {gpu.pp_rank}, "
                           f"but save requested tp_rank {tp_rank}, pp_rank {pp_rank}")
        ctxs = []
        wanted = set()
        for layer_name, block_ids, block_hashes in saves:
            if len(block_ids) != len(block_hashes):
                raise _invalid(f"block_ids length {len(block_ids)} does not match block_hashes {len(block_hashes)} "
                               f"for layer {layer_name}")
            lid = topo.layer_id(layer_name)
            lay = gpu.layouts.get(layer_name)
            if lay is None:
                raise _invalid(f"layer {layer_name} not registered on device")
            slot = topo.slot_index(lid, tp_rank)
            grp = topo.layer_group[lid]
            blocks = []
            for idx, h in zip(block_ids, block_hashes):
                if idx >= lay.num_blocks:
                    raise _invalid(f"block_id {idx} out of range (num_blocks={lay.num_blocks}) for layer "
                                   f"{layer_name}")
                blocks.append((int(idx), bytes(h)))
            if not blocks:
                continue
            for _, h in blocks:
                wanted.add((grp, h))
            ctxs.append(dict(name=layer_name, layout=lay, slot=slot, group=grp, blocks=blocks, raw=[]))
        if not ctxs:
            return
        # phase 1: drop hashes already sealed in the read cache (per group)
        wanted = {(g, h) for (g, h) in wanted if (inst.namespace, po.group_hash(h, g)) not in self.read_cache}
        if not wanted:
            return
        for c in ctxs:
            c["blocks"] = [(i, h) for (i, h) in c["blocks"] if (c["group"], h) in wanted]
        ctxs = [c for c in ctxs if c["blocks"]]
        if not ctxs:
            return
        # phase 2: host placement
        page_first = topo.page is not None
        tasks = []
        pages: List[_Alloc] = []
        if page_first:
            shard = ctxs[0]["slot"]
            page_size = topo.page["shard_page_sizes"][shard]
            ref_blocks = ctxs[0]["blocks"]
            for c in ctxs:
                if c["layout"].is_split:
                    raise _invalid(f"page-first save does not support split K/V (layer {c['name']})")
                if c["slot"] != shard:
                    raise _invalid("page-first save spans multiple shards (one writer must save one shard)")
                if c["blocks"] != ref_blocks:
                    raise _invalid("page-first save requires the same block set across all layers")
            ids = sorted({topo.layer_id(c["name"]) for c in ctxs})
            shard_layers = sum(1 for s in topo.page["layer_shard"] if s == shard)
            if len(ids) != shard_layers:
                raise _invalid(f"page-first save must cover all {shard_layers} layers of shard {shard}, got "
                               f"{len(ids)} distinct (one worker must write a shard's entire page)")
            if page_size == 0:
                raise EngineError("Storage", "page size is zero")
            for _ in ref_blocks:
                a = self.pool.allocate(page_size)
                if a is None:
                    raise EngineError("Storage", "pinned pool exhausted while allocating page")
                pages.append(a)
            for c in ctxs:
                off, _nbytes = topo.page_placement(topo.layer_id(c["name"]))
                blocks = [(idx, [po.HostSeg(pg.host + off, pg.host + off, pg.ident)], 0)
                          for (idx, _), pg in zip(c["blocks"], pages)]
                tasks.append((c["layout"], blocks))
        else:
            for c in ctxs:
                lay = c["layout"]
                n = len(c["blocks"])
                n_allocs, per = (n, 1) if self.blockwise else (1, n)
                raw: List[_RawBlock] = []
                for _ in range(n_allocs):
                    if lay.is_split:
                        stride = lay.padded_segment_bytes
                        ka = self._alloc(stride * per, "K segment buffer")
                        va = self._alloc(stride * per, "V segment buffer")
                        for i in range(per):
                            raw.append(_RawBlock([_Segment(ka, i * stride, stride), _Segment(va, i * stride, stride)]))
                    else:
                        stride = lay.padded_block_bytes
                        a = self._alloc(stride * per, "block buffer")
                        for i in range(per):
                            raw.append(_RawBlock([_Segment(a, i * stride, stride)]))
                c["raw"] = raw
                blocks = [(idx, [po.HostSeg(s.host, s.host, s.alloc.ident) for s in rb.segments], 0)
                          for (idx, _), rb in zip(c["blocks"], raw)]
                tasks.append((lay, blocks))
        # phase 3: one descriptor batch, device -> host
        descs, n, _total = po.build_copy_descs(tasks)
        po.execute(descs, n, host_is_src=False)
        # phase 4: group slots by hash, seal complete blocks
        if page_first:
            slot = ctxs[0]["slot"]
            psize = topo.page["shard_page_sizes"][slot]
            for (_, h), pg in zip(ctxs[0]["blocks"], pages):
                self._insert(inst.namespace, h, slot, _RawBlock([_Segment(pg, 0, psize)]), topo.total_slots())
        else:
            for c in ctxs:
                total = topo.group_total_slots(c["group"])
                for (_, h), rb in zip(c["blocks"], c["raw"]):
                    self._insert(inst.namespace, po.group_hash(h, c["group"]), c["slot"], rb, total)

    def _insert(self, namespace, key_hash, slot, raw, total_slots):
        """storage/write_path.rs:119-254: late duplicates are dropped, a block becomes visible
        only once every slot has arrived."""
        key = (namespace, key_hash)
        if key in self.read_cache:
            self._release(raw)
            return
        if key not in self.inflight:
            self.inflight_born[key] = time.monotonic()
        total, slots = self.inflight.setdefault(key, (total_slots, {}))
        if total != total_slots:
            return
        if slot in slots:
            self._release(raw)
            return
        slots[slot] = raw
        if len(slots) == total:
            del self.inflight[key]
            self.inflight_born.pop(key, None)
            self.read_cache[key] = SealedBlock([slots[i] for i in range(total)])

    def _release(self, raw: _RawBlock):
        pass  # the model never reuses pool memory of dropped duplicates; offsets are not part of the contract

    def flush_saves(self):
        pass

    # -- query / leases ------------------------------------------------------------------------
    def query_prefix(self, instance_id, hashes: Sequence[bytes]):
        """lib.rs:506-533 + read_cache.rs:64-80: longest cached prefix; returns (blocks, missing)."""
        inst = self._instance(instance_id)
        blocks = []
        for h in hashes:
            b = self.read_cache.get((inst.namespace, bytes(h)))
            if b is None:
                break
            blocks.append(b)
        return blocks, len(hashes) - len(blocks)

    def query_group_membership(self, instance_id, group_id, hashes):
        inst = self._instance(instance_id)
        self._sealed(inst).group_total_slots(group_id)
        return [self.read_cache.get((inst.namespace, po.group_hash(bytes(h), group_id))) for h in hashes]

    def create_query_lease(self, instance_id, blocks) -> bytes:
        inst = self._instance(instance_id)
        if not blocks:
            raise _invalid("query lease requires at least one block")
        token = os.urandom(16)
        self.leases[token] = [instance_id, list(blocks), max(1, inst.world_size)]
        return token

    def release_query_lease(self, lease: bytes) -> bool:
        return self.leases.pop(bytes(lease), None) is not None

    def _consume(self, instance_id, lease):
        ent = self.leases.get(bytes(lease))
        if ent is None:
            raise EngineError("Storage", "query lease is unknown or expired")
        if ent[0] != instance_id:
            raise EngineError("Storage", f"query lease belongs to instance {ent[0]}, got {instance_id}")
        if ent[2] > 1:
            ent[2] -= 1
            return list(ent[1])
        del self.leases[bytes(lease)]
        return ent[1]

    # -- load: lib.rs:715-895 -------------------------------------------------------------------
    def batch_load(self, instance_id, tp_rank, device_id, layer_groups: Sequence[Sequence[str]],
                   loads: Sequence[Tuple[bytes, Sequence[Sequence[Optional[int]]]]]):
        inst = self._instance(instance_id)
        topo = self._sealed(inst)
        gpu = inst.gpus.get(device_id)
        if gpu is None:
            raise EngineError("WorkerMissing", instance_id, device_id)
        if not layer_groups:
            raise _invalid("load requires at least one layer group")
        flat = [nm for grp in layer_groups for nm in grp]
        if len(set(flat)) != len(flat):
            raise _invalid("load layer names must be unique across groups")
        storage_group: List[Optional[int]] = []
        for names in layer_groups:
            g = None
            for nm in names:
                lg = topo.layer_group[topo.layer_id(nm)]
                if g is None:
                    g = lg
                elif g != lg:
                    raise _invalid(f"load group mixes storage groups {g} and {lg} (layer {nm})")
            storage_group.append(g)
        targets: List[List[Tuple[int, int]]] = [[] for _ in layer_groups]
        cache: List[SealedBlock] = []
        for lease, ids_by_group in loads:
            blocks = self._consume(instance_id, lease)
            if len(ids_by_group) != len(layer_groups):
                raise _invalid(f"load group count {len(ids_by_group)} does not match layer group count "
                               f"{len(layer_groups)}")
            start = len(cache)
            for gi, tg in enumerate(ids_by_group):
                if len(blocks) != len(tg):
                    raise _invalid(f"query lease block count {len(blocks)} does not match destination block count "
                                   f"{len(tg)} for group {gi}")
                if storage_group[gi] is not None:
                    expected = topo.group_total_slots(storage_group[gi])
                    for si, dst in enumerate(tg):
                        if dst is not None and len(blocks[si].slots) != expected:
                            raise _invalid(
                                f"stored block has {len(blocks[si].slots)} slots but storage group "
                                f"{storage_group[gi]} of instance {instance_id} expects {expected}: namespace is "
                                "shared by incompatible KV layouts")
                targets[gi].extend((dst, start + si) for si, dst in enumerate(tg) if dst is not None)
            cache.extend(blocks)
        tasks = []
        for gi, names in enumerate(layer_groups):
            for nm in names:
                lid = topo.layer_id(nm)
                lay = gpu.layouts.get(nm)
                if lay is None:
                    raise _invalid(f"layer {nm} not registered on device {device_id}")
                slot = topo.slot_index(lid, tp_rank)
                pp = topo.page_placement(lid)
                off = pp[0] if pp else 0
                blocks = []
                for dst, si in targets[gi]:
                    raw = cache[si].get_slot(slot)
                    if raw is None:
                        raise _invalid(f"stored block is missing slot {slot} for layer {nm}")
                    segs = [po.HostSeg(s.host, s.host, s.alloc.ident) for s in raw.segments]
                    blocks.append((dst, segs, off))
                if blocks:
                    tasks.append((lay, blocks))
        if not tasks:
            return
        descs, n, _ = po.build_copy_descs(tasks)
        po.execute(descs, n, host_is_src=True)

    # -- introspection used by the parity tests ----------------------------------------------------
    def block_slot_image(self, instance_id, raw_hash, slot, group=0) -> Optional[List[bytes]]:
        inst = self._instance(instance_id)
        b = self.read_cache.get((inst.namespace, po.group_hash(bytes(raw_hash), group)))
        if b is None:
            return None
        raw = b.get_slot(slot)
        return None if raw is None else [s.bytes() for s in raw.segments]
