"""N > 1 on CPU: two gloo ranks plan their shards and time a run the way bench.py does; the oracle
engine model seals a TP=2 block only once both ranks have saved their slots."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle.engine_model import OracleEngine
from pegaflow_b200 import sharding
from tests import scenarios as sc


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        plan = sharding.rank_plan(rank, world, n_layers=4, payload_bytes_per_rank=1 << 20)
        gathered = [None] * world
        dist.all_gather_object(gathered, (plan.seed, plan.slots, plan.device))
        slots = sorted(s for _, sl, _ in gathered for s in sl)
        assert slots == list(range(4 * world)), "the ranks' slots must partition the slot space"
        assert len({g[0] for g in gathered}) == world and [g[2] for g in gathered] == list(range(world))
        elapsed = sharding.barrier_and_max(0.5 + rank, device="cpu")
        assert elapsed == 0.5 + (world - 1)
        agg = sharding.aggregate_throughput([10 ** 9] * world, elapsed)
        # two instances on one box: rank 0 is instance A and hands its "regions" to rank 1, its partner
        who = sharding.peer_role(rank, world)
        everyone = [None] * world
        dist.all_gather_object(everyone, [b"region-of-%d" % rank] if who.role == "A" else None)
        if who.role == "B":
            assert everyone[who.partner] == [b"region-of-%d" % who.partner] and who.pair == who.partner
        else:
            assert who.role == "A" and everyone[who.partner] is None
        np.save(os.path.join(out_dir, f"r{rank}.npy"), np.array([agg]))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_plan_disjoint_shards_and_time_like_the_bench(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    vals = [float(np.load(tmp_path / f"r{r}.npy")[0]) for r in range(world)]
    assert vals[0] == vals[1] == pytest.approx(2 / 1.5)


def test_rank_plan_and_peer_roles():
    with pytest.raises(ValueError):
        sharding.rank_plan(2, 2, n_layers=1, payload_bytes_per_rank=1)
    roles = [sharding.peer_role(r, 8) for r in range(8)]
    assert [x.role for x in roles] == ["A"] * 4 + ["B"] * 4
    assert [x.partner for x in roles] == [4, 5, 6, 7, 0, 1, 2, 3] and [x.pair for x in roles] == [0, 1, 2, 3] * 2
    assert [sharding.peer_role(r, 3).role for r in range(3)] == ["A", "B", None]
    assert sharding.peer_role(0, 1).role is None


def test_tp2_block_seals_only_when_both_ranks_saved_and_loads_per_rank():
    """instance.rs:251-269 + write_path.rs:186-254 on the oracle: slot = layer * tp_size + tp_rank."""
    eng, mem = OracleEngine(16 << 20), sc.NumpyMem()
    layers = {r: [sc.Layer(f"l{i}", 8, 1024) for i in range(2)] for r in range(2)}
    for r in range(2):
        sc.register(eng, mem, "tp", "ns", layers[r], device_id=r, tp_rank=r, tp_size=2, world_size=2)
        for i, L in enumerate(layers[r]):
            mem.write(L.buf, sc.fill_pattern(8, 1024, 0x10 * (2 * r + i)))
    h = sc.make_block_hashes(3, 1)
    eng.batch_save("tp", 0, 0, 0, [(L.name, [1, 2, 3], h) for L in layers[0]])
    assert eng.query_prefix("tp", h) == ([], 3)
    eng.batch_save("tp", 1, 0, 1, [(L.name, [4, 5, 6], h) for L in layers[1]])
    blocks, missing = eng.query_prefix("tp", h)
    assert missing == 0 and len(blocks[0].slots) == 4
    assert eng.block_slot_image("tp", h[0], 0)[0] == bytes([2]) * 1024           # l0, rank 0, block 1
    assert eng.block_slot_image("tp", h[0], 3)[0] == bytes([5 + 0x30]) * 1024    # l1, rank 1, block 4
    lease = eng.create_query_lease("tp", blocks)
    for r in range(2):
        for L in layers[r]:
            mem.zero(L.buf)
        eng.batch_load("tp", r, r, [[L.name for L in layers[r]]], [(lease, [[0, 1, 2]])])
    assert not eng.release_query_lease(lease), "the second consumer used the lease up"
    assert mem.read(layers[1][1].buf)[:1024].tolist() == [5 + 0x30] * 1024
