"""The multi-replica path on CPU: two gloo ranks split one request list the way bench.py does under
torchrun (same partition on every rank, disjoint shards, results merged by request id, timing reduced
as the maximum over ranks)."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mini_vllm_b200.dispatcher import merge_outputs, partition_by_tokens
from mini_vllm_b200.workloads import config2_requests, config5_requests


def test_partition_is_balanced_deterministic_and_complete():
    reqs = config5_requests(seed=0, n=512)
    costs = [len(r.prompt) + r.max_tokens for r in reqs]
    for n in (1, 2, 4, 8):
        parts = partition_by_tokens(costs, n)
        assert sorted(i for p in parts for i in p) == list(range(len(costs)))
        loads = [sum(costs[i] for i in p) for p in parts]
        assert max(loads) - min(loads) <= max(costs)
        assert parts == partition_by_tokens(costs, n)
    outs = merge_outputs(parts, [[f"r{i}" for i in p] for p in parts], len(costs))
    assert outs == [f"r{i}" for i in range(len(costs))]
    with pytest.raises(ValueError):
        merge_outputs(parts, [[] for _ in parts], len(costs))


def _rank_main(rank: int, world: int, port: int, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        reqs = config2_requests(seed=0, n=64 * world)
        costs = [len(r.prompt) + r.max_tokens for r in reqs]
        mine = partition_by_tokens(costs, world)[rank]
        # "generate": a stand-in result that depends only on the request
        results = [sum(reqs[i].prompt) % 9973 for i in mine]
        gathered = [None] * world
        dist.all_gather_object(gathered, (mine, results))
        merged = merge_outputs([g[0] for g in gathered], [g[1] for g in gathered], len(reqs))
        assert merged == [sum(r.prompt) % 9973 for r in reqs]
        # timing contract of the bench: value = all tokens / max over ranks
        stats = torch.tensor([10.0 + rank, float(sum(costs[i] for i in mine))], dtype=torch.float64)
        mx, sm = stats.clone(), stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        assert mx[0].item() == 10.0 + world - 1 and sm[1].item() == float(sum(costs))
        ret[rank] = len(mine)
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_split_and_merge():
    world, port = 2, 29731
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_rank_main, args=(world, port, ret), nprocs=world, join=True)
        assert sum(ret.values()) == 64 * world and abs(ret[0] - ret[1]) <= 16
