"""World-size-2 checks of the multi-GPU exchange logic on CPU (gloo backend)."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from worldattention_b200 import sharded
        # ragged all-gather: rank r contributes r + 1 blocks of pooled keys
        sizes = [r + 1 for r in range(world)]
        local = torch.full((1, 2, sizes[rank], 4), float(rank))
        full = sharded.all_gather_cat(local, 2, sizes=sizes)
        assert full.shape == (1, 2, sum(sizes), 4)
        assert full[0, 0, :, 0].tolist() == [float(r) for r in range(world) for _ in range(sizes[r])]
        # equal-size all-gather of packed partials along a new leading axis
        part = torch.full((1, 6, 3), float(rank + 1))
        assert sharded.all_gather_cat(part, 0).shape == (world, 6, 3)
        # head-split outputs return in head order even for an interleaved plan
        plan = [[0, 3], [1, 2]]
        mine = torch.stack([torch.full((1, 5, 2), float(h)) for h in plan[rank]], dim=2)      # [B, L, H_local, D]
        gathered = sharded.gather_heads(mine, plan)
        assert gathered.shape == (1, 5, 4, 2)
        assert gathered[0, 0, :, 0].tolist() == [0.0, 1.0, 2.0, 3.0]
        # every rank derives the same shard plan and head plan
        shards = sharded.plan_kv_shards(32760, 128, world, 1560)
        blob = [None] * world
        dist.all_gather_object(blob, (shards, sharded.plan_head_split(12, world, [4, 8, 16, 32] * 3)))
        assert all(b == blob[0] for b in blob)
        # the row exchange of the KV-sharded forward: rank j receives rows [j * rp, (j + 1) * rp) of every shard's records
        q_len, heads, rec = 7, 2, 5                      # ragged: 4 + 3 rows
        rp, row_plan = sharded.exchange_rows(q_len, world)
        assert (rp, row_plan) == (4, [(0, 4), (4, 3)])
        records = torch.zeros((rp * world, heads, rec))
        records[:q_len] = (rank * 1000 + torch.arange(q_len, dtype=torch.float32)).view(-1, 1, 1)
        recv = torch.empty_like(records)
        dist.all_to_all_single(recv, records)
        got = recv.view(world, rp, heads, rec)
        first, count = row_plan[rank]
        for shard in range(world):
            assert got[shard, :count, 0, 0].tolist() == [shard * 1000.0 + first + r for r in range(count)]
        rows = torch.full((rp, heads, 3), -1.0)
        rows[:count] = (first + torch.arange(count, dtype=torch.float32)).view(-1, 1, 1)
        full = torch.empty((world * rp, heads, 3))
        dist.all_gather_into_tensor(full, rows)
        assert full[:q_len, 0, 0].tolist() == [float(r) for r in range(q_len)]
        results[rank] = "ok"
    finally:
        dist.destroy_process_group()


def test_exchange_logic_world_size_2():
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    assert dict(results) == {0: "ok", 1: "ok"}
