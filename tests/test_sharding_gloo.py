"""Host logic of the multi-GPU path on CPU: the (batch x KV head) partition and the
max-over-ranks reduction, with two gloo ranks."""
import os

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flash_attention3_b200 import sharding


def test_plan_is_a_disjoint_contiguous_cover():
    for batch, hkv in [(16, 32), (2, 8), (1, 4), (3, 5), (1, 1), (7, 2)]:
        for world in (1, 2, 3, 4, 8):
            seen = np.zeros((batch, hkv), dtype=int)
            last = -1
            for shards in sharding.plan(batch, hkv, world):
                for s in shards:
                    assert s.batch_count == 1 or (s.kv_head_begin == 0 and s.kv_head_count == hkv)
                    seen[s.batch_begin:s.batch_begin + s.batch_count,
                         s.kv_head_begin:s.kv_head_begin + s.kv_head_count] += 1
                    first = s.batch_begin * hkv + s.kv_head_begin
                    assert first > last  # ranks and shards come in ascending unit order
                    last = first
            assert (seen == 1).all()
            sizes = [sum(s.batch_count * s.kv_head_count for s in sh) for sh in sharding.plan(batch, hkv, world)]
            assert max(sizes) - min(sizes) <= 1


def test_benchmark_shapes():
    # B=16,H=32 over 8 GPUs: two whole batches each; B=2,Hkv=8 over 8: two KV heads each; H=4 over 4: one head
    assert sharding.plan(16, 32, 8)[3] == [sharding.Shard(6, 2, 0, 32)]
    assert sharding.plan(2, 8, 8)[5] == [sharding.Shard(1, 1, 2, 2)]
    assert sharding.plan(1, 4, 4)[2] == [sharding.Shard(0, 1, 2, 1)]


def test_shard_views_are_contiguous_byte_ranges():
    b, hq, hkv, s, d = 3, 8, 4, 16, 8
    q = torch.arange(b * hq * s * d).reshape(b, hq, s, d)
    k = torch.arange(b * hkv * s * d).reshape(b, hkv, s, d)
    lse = torch.arange(b * hq * s).reshape(b, hq, s)
    for shards in sharding.plan(b, hkv, 5):
        for sh in shards:
            (qv,), (kv,), (lv,) = sharding.slice_tensors(sh, hq // hkv, [q], [k], [lse])
            for view in (qv, kv, lv):
                assert view.is_contiguous()
                flat = view.reshape(-1)
                assert int(flat[-1] - flat[0]) == flat.numel() - 1  # one unbroken range of the parent


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    shards = sharding.plan(2, 8, world)[rank]
    units = sum(s.batch_count * s.kv_head_count for s in shards)
    total = torch.tensor([units])
    dist.all_reduce(total)
    slowest = sharding.max_over_ranks(10.0 + rank, dist)
    dist.barrier()
    results[rank] = (int(total.item()), slowest)
    dist.destroy_process_group()


def test_two_gloo_ranks_cover_the_problem_and_agree_on_the_slowest():
    world, port = 2, 29500 + os.getpid() % 2000
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        assert dict(results) == {0: (16, 11.0), 1: (16, 11.0)}
