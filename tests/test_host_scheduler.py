"""Block manager and scheduler against traces recorded from the reference's own classes."""
import json
from pathlib import Path
from types import SimpleNamespace

import pytest

from mini_vllm_b200.config import SamplingParams
from mini_vllm_b200.engine.request import Request
from mini_vllm_b200.kvcache.block_manager import KVCacheBlock, KVCacheBlockManager
from mini_vllm_b200.scheduler.batch import Batch
from mini_vllm_b200.scheduler.scheduler import Scheduler

GOLD = Path(__file__).parent / "golden"


def test_block_hash_known_answers():
    h = json.loads((GOLD / "hashes.json").read_text())
    for kat in h["kat"]:
        assert KVCacheBlock.compute_hash(kat["tokens"], kat["prefix"]) == kat["hash"]
    # two known answers of the chained xxh64 block hash (block_manager.py:17-27) computed with xxhash 3.x
    assert KVCacheBlock.compute_hash([1, 2, 3]) == 0xb5148cb100a911fc
    assert KVCacheBlock.compute_hash([1, 2, 3], 7) == 0xc0618d2457d05e39
    m = KVCacheBlockManager(10240, 256)
    r = Request(list(range(600)))
    m.allocate_blocks_for_prefill(r)
    assert r.blocks == h["fresh_pool_first_ids"] == [10239, 10238, 10237]


def test_block_manager_trace_matches_reference():
    t = json.loads((GOLD / "block_manager.json").read_text())
    m = KVCacheBlockManager(t["capacity"], t["block_size"], support_prefix_cache=True)
    live = []
    for ev in t["events"]:
        if ev["op"] == "alloc":
            r = Request(ev["tokens"])
            assert m.can_allocate_new_block(r) == ev["can"]
            if ev["can"]:
                m.allocate_blocks_for_prefill(r)
                r.state = Request.RUNNING
                live.append(r)
                assert r.blocks == ev["blocks"] and r.num_cached_tokens == ev["cached"]
        elif ev["op"] == "grow":
            r = live[ev["index"]]
            for tok, nb in zip(ev["tokens"], ev["nblocks_after_each"]):
                r.append_output_token(tok)
                m.cache_block_if_needed(r)
                if m.can_allocate_new_block(r):
                    m.allocate_block_for_decode(r)
                assert len(r.blocks) == nb
            assert r.blocks == ev["blocks"]
        else:
            m.deallocate(live[ev["index"]])
        assert m.free_block_ids == ev["free_ids"]
        assert sorted(m.used_block_ids) == ev["used_ids"]


def test_reference_unit_test_body_with_prefix_cache():
    """tests/test_block_manager.py of the reference (passes there only with the prefix cache on)."""
    import random
    rnd = random.Random(0)
    m = KVCacheBlockManager(10240, 256, support_prefix_cache=True)
    tokens = [rnd.randint(1, 25600) for _ in range(25600)]
    req = Request(tokens)
    m.allocate_blocks_for_prefill(req)
    assert len(req.blocks) == 100 == len(m.hash_to_block_id) == len(m.used_block_ids)
    held = []
    for i in range(1, 100):
        r = Request(tokens[:i * 256])
        if not m.can_allocate_new_block(r):
            for x in held:
                m.deallocate(x)
            held.clear()
        m.allocate_blocks_for_prefill(r)
        assert len(r.blocks) == i and r.num_cached_tokens == len(r.tokens)
        held.append(r)


def test_fully_cached_prompt_keeps_a_query_token_when_asked():
    m = KVCacheBlockManager(16, 256, support_prefix_cache=True, keep_last_block_uncached=True)
    a = Request(list(range(512)))
    m.allocate_blocks_for_prefill(a)
    b = Request(list(range(512)))
    m.allocate_blocks_for_prefill(b)
    assert b.num_cached_tokens == 256 and b.blocks[0] == a.blocks[0] and b.blocks[1] != a.blocks[1]


@pytest.mark.parametrize("name", ["roomy", "tight_preempt", "prefix_cache"])
def test_scheduler_trace_matches_reference(name):
    t = json.loads((GOLD / "scheduler.json").read_text())[name]
    cfg = SimpleNamespace(max_num_batched_seqs=t["max_seqs"], max_num_batched_tokens=t["max_tokens"],
                          eos_token_ids={9999}, kv_cache_num_blocks=t["capacity"], kv_cache_block_size=256,
                          enable_prefix_cache=False)
    sch = Scheduler(cfg)
    if t["prefix_cache"]:
        sch.block_manager.support_prefix_cache = True      # reference behaviour, including full hits
    reqs = [Request(p, SamplingParams(max_tokens=sp["max_tokens"], ignore_eos=sp["ignore_eos"]))
            for p, sp in zip(t["prompts"], t["sampling"])]
    base = reqs[0].id
    for r in reqs:
        sch.submit(r)
    for step in t["steps"]:
        batch = sch.schedule()
        assert batch is not None and batch.type == step["type"]
        rows = [{"rid": r.id - base, "len": len(r.tokens), "cached": r.num_cached_tokens, "blocks": list(r.blocks)}
                for r in batch.requests]
        assert rows == step["rows"]
        sch.update(batch, step["tokens"])
        assert [r.id - base for r in sch.waiting] == step["waiting"]
        assert [r.id - base for r in sch.running] == step["running"]
    assert sch.finished
    assert [r.completion_tokens for r in reqs] == t["completions"]
    assert any(s["type"] == Batch.DECODE for s in t["steps"])


def test_mixed_steps_admit_prompts_next_to_running_decodes():
    """With ``enable_mixed_steps`` a step may hold prompts followed by decoding requests; every request
    still produces exactly its tokens, the caps hold, and without the flag nothing changes."""
    import random
    rnd = random.Random(7)
    prompts = [[rnd.randrange(1000) for _ in range(rnd.randrange(5, 600))] for _ in range(40)]
    budgets = [rnd.randrange(3, 40) for _ in prompts]

    def run(mixed):
        cfg = SimpleNamespace(max_num_batched_seqs=8, max_num_batched_tokens=1024, eos_token_ids=set(),
                              kv_cache_num_blocks=24, kv_cache_block_size=256, enable_prefix_cache=False,
                              enable_mixed_steps=mixed)
        sch = Scheduler(cfg)
        reqs = [Request(p, SamplingParams(max_tokens=m, ignore_eos=True)) for p, m in zip(prompts, budgets)]
        for r in reqs:
            sch.submit(r)
        kinds, steps = set(), 0
        while not sch.finished:
            batch = sch.schedule()
            assert batch is not None
            kinds.add(batch.type)
            b, nd = len(batch.requests), batch.num_decode
            assert 0 < b <= 8
            if batch.type == Batch.MIXED:
                assert 0 < nd < b
                new_tokens = sum(len(r.tokens) - r.num_cached_tokens for r in batch.requests[:b - nd]) + nd
                assert new_tokens <= 1024
                assert all(r.num_completion_tokens == 0 for r in batch.requests[:b - nd])
                assert all(r.num_completion_tokens > 0 for r in batch.requests[b - nd:])
                assert len({r.id for r in batch.requests}) == b
            # every scheduled request owns the blocks its tokens need
            assert all(len(r.blocks) * 256 >= len(r.tokens) for r in batch.requests)
            sch.update(batch, [1] * b)
            steps += 1
        assert [r.num_completion_tokens for r in reqs] == budgets
        return kinds, steps

    kinds, steps = run(True)
    assert Batch.MIXED in kinds
    plain_kinds, plain_steps = run(False)
    assert Batch.MIXED not in plain_kinds
    assert steps < plain_steps                              # prompts no longer cost steps of their own


def test_stop_ends_a_running_or_a_preempted_request():
    """``Scheduler.stop`` (used when an EOS is learnt of late): blocks go back, queues forget the request."""
    cfg = SimpleNamespace(max_num_batched_seqs=4, max_num_batched_tokens=4096, eos_token_ids=set(),
                          kv_cache_num_blocks=8, kv_cache_block_size=256, enable_prefix_cache=False)
    sch = Scheduler(cfg)
    reqs = [Request(list(range(300)), SamplingParams(max_tokens=50, ignore_eos=True)) for _ in range(3)]
    for r in reqs:
        sch.submit(r)
    batch = sch.schedule()
    assert batch.type == Batch.PREFILL and len(batch.requests) == 3
    sch.update(batch, [1, 1, 1])
    free_before = len(sch.block_manager.free_block_ids)
    sch.stop(reqs[0])
    assert reqs[0].finished and reqs[0] not in sch.running
    assert len(sch.block_manager.free_block_ids) == free_before + 2
    sch.preempt(reqs[2]); sch.running.remove(reqs[2])
    assert reqs[2] in sch.waiting
    sch.stop(reqs[2])
    assert reqs[2].finished and reqs[2] not in sch.waiting
    while not sch.finished:
        b = sch.schedule()
        assert [r.id for r in b.requests] == [reqs[1].id]
        sch.update(b, [1])
    assert reqs[1].num_completion_tokens == 50
