"""Host-side plan of a multi-GPU run: the path shards by rank with no data exchange.

Rank r owns GPU r of the node, its own transfer workers and stream, a pinned pool on that GPU's
NUMA node, and the storage slots ``(layer, tp_rank = r)`` (pegaflow-core/src/instance.rs:251-269,
gpu_worker.rs:131-201).  The only collective is the one that times a run: a barrier and a
max-over-ranks of the elapsed time.  Where two instances share a box (same-box prefix hits over
NVLink), the first half of the ranks is one instance and the second half the other, paired rank
by rank.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence


@dataclass(frozen=True)
class RankPlan:
    rank: int
    world: int
    device: int
    seed: int
    slots: List[int]        # storage slots this rank writes, layer-first: layer * tp_size + rank
    pool_bytes: int


def rank_plan(rank: int, world: int, *, n_layers: int, payload_bytes_per_rank: int, base_seed: int = 42,
              config_index: int = 2, local_rank: int | None = None) -> RankPlan:
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} out of range (world {world})")
    return RankPlan(rank=rank, world=world, device=rank if local_rank is None else local_rank,
                    seed=base_seed + config_index + rank, slots=[l * world + rank for l in range(n_layers)],
                    pool_bytes=payload_bytes_per_rank + (64 << 20))


@dataclass(frozen=True)
class PeerRole:
    role: Optional[str]     # "A" (owns the prefix), "B" (pulls it), None (odd rank out)
    pair: int               # index of the rank-aligned pair
    partner: Optional[int]  # rank of the other side


def peer_role(rank: int, world: int) -> PeerRole:
    """Two instances of the same TP degree on one box: ranks 0 .. world/2-1 are instance A, ranks
    world/2 .. 2*(world/2)-1 instance B; B's rank i pulls from A's rank i (rank-aligned shards, so no
    exchange between pairs).  With an odd world the last rank takes no part."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} out of range (world {world})")
    half = world // 2
    if rank < half:
        return PeerRole("A", rank, rank + half)
    if rank < 2 * half:
        return PeerRole("B", rank - half, rank - half)
    return PeerRole(None, -1, None)


def aggregate_throughput(bytes_per_rank: Sequence[int], elapsed_max_seconds: float) -> float:
    """Whole-job GB/s: everything all ranks moved, over the slowest rank's time."""
    return sum(bytes_per_rank) / elapsed_max_seconds / 1e9


def barrier_and_max(value: float, group=None, device=None) -> float:
    """Barrier, then the max of `value` over the ranks of `group` (works on NCCL and gloo)."""
    import torch
    import torch.distributed as dist

    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device or "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
