"""The engine's pipelined step loop against the plain step loop, on a stand-in executor (no GPU): sampled
tokens reach the host late, requests stop on EOS, the pool is tight enough for preemptions, steps may be
mixed - the completions must be the same as when every step is waited for."""
import copy
import random
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from mini_vllm_b200.config import SamplingParams
from mini_vllm_b200.engine.engine import Engine
from mini_vllm_b200.engine.metrics import Metrics
from mini_vllm_b200.scheduler.batch import Batch
from mini_vllm_b200.scheduler.scheduler import Scheduler


def next_token(prompt_sum: int, position: int) -> int:
    """What the stand-in model emits after ``position`` tokens: a function of the prompt and the position
    only, so that speculative steps past an EOS cannot leak into what is kept."""
    return (prompt_sum * 31 + position * 17 + (position * position) % 11) % 50


class LateEvent:
    def __init__(self, fire):
        self.fire = fire

    def synchronize(self):
        self.fire()


class StandInExecutor:
    """``execute`` answers at once; ``launch`` fills its host buffer only when the event is waited for, and
    reads decode inputs from the device-side table the way the real packing kernel does (so a decode step
    launched with a placeholder on the host still sees the real previous token)."""

    def __init__(self):
        self.table = {}
        self.launched = []
        self.status_checked = 0

    def ensure_token_table(self, n):
        pass

    def check_device_status(self):
        self.status_checked += 1

    @staticmethod
    def _tokens(batch):
        out = []
        for r in batch.requests:
            psum = sum(r.tokens[:r.prompt_token_count])
            out.append(next_token(psum, len(r.tokens)))
        return out

    def execute(self, batch):
        for r in batch.requests:
            assert min(r.tokens) >= 0, "a step that needs real tokens saw a placeholder"
        return self._tokens(batch)

    def launch(self, batch, slots):
        self.launched.append(batch.type)
        if batch.type != Batch.DECODE:                 # prompts (and mixed steps) are packed from the host's tokens
            n_host = len(batch.requests) - (batch.num_decode if batch.type == Batch.MIXED else 0)
            for r in batch.requests[:n_host] if batch.type == Batch.MIXED else batch.requests:
                assert min(r.tokens) >= 0, "a prefill was launched over placeholder tokens"
            if batch.type == Batch.MIXED:
                for r in batch.requests[n_host:]:
                    assert r.tokens[-1] >= 0, "a mixed step's decode input was a placeholder"
        toks = self._tokens(batch)
        host = torch.zeros(len(toks), dtype=torch.int64)
        for s, t in zip(slots.tolist(), toks):
            self.table[s] = t
        return host, LateEvent(lambda: host.copy_(torch.tensor(toks)))


def make_engine(mixed: bool, blocks: int, prefix: bool = False):
    cfg = SimpleNamespace(max_num_batched_seqs=5, max_num_batched_tokens=2048, eos_token_ids={0, 7, 13, 21, 34},
                          kv_cache_num_blocks=blocks, kv_cache_block_size=256, enable_prefix_cache=prefix,
                          enable_mixed_steps=mixed)
    eng = object.__new__(Engine)
    eng.config, eng.tokenizer = cfg, None
    eng.executor, eng.scheduler, eng.metrics = StandInExecutor(), Scheduler(cfg), Metrics()
    return eng


@pytest.mark.parametrize("mixed", [False, True])
@pytest.mark.parametrize("blocks", [40, 7])
def test_pipelined_loop_gives_the_plain_loop_completions(mixed, blocks):
    rnd = random.Random(3 + blocks)
    prompts = [[rnd.randrange(1, 50) for _ in range(rnd.randrange(3, 400))] for _ in range(24)]
    params = [SamplingParams(max_tokens=rnd.randrange(2, 45), ignore_eos=(i % 5 == 4)) for i in range(len(prompts))]

    plain = make_engine(mixed, blocks)
    reqs = [plain.submit(p, sp) for p, sp in zip(prompts, copy.deepcopy(params))]
    while not plain.finished:
        plain.step()
    want = [r.completion_tokens for r in reqs]
    eos = plain.config.eos_token_ids
    assert any(len(w) < sp.max_tokens for w, sp in zip(want, params)), "no request stopped on EOS"
    assert all(len(w) == sp.max_tokens for w, sp in zip(want, params) if sp.ignore_eos)

    piped = make_engine(mixed, blocks)
    assert piped._schedule_is_token_independent(params)
    out = piped.generate(prompts, copy.deepcopy(params), use_tqdm=False)
    got = [o["tokens"] for o in out]
    assert got == want
    assert all(t not in eos for toks, sp in zip(got, params) if not sp.ignore_eos for t in toks[:-1])
    assert piped.executor.status_checked == 1
    assert piped.scheduler.finished
    bm = piped.scheduler.block_manager
    assert len(bm.free_block_ids) == blocks, "blocks leaked"
    if mixed:
        assert Batch.MIXED in piped.executor.launched


def test_pipelined_loop_with_prefix_cache():
    """Prefix caching under the pipelined loop: blocks that fill up with generated tokens are published when
    those tokens are known.  Prompts share 512-token prefixes, and follow-up prompts repeat an earlier
    request's prompt plus its completion (a second turn), so hits on generated blocks matter."""
    rnd = random.Random(11)
    shared = [rnd.randrange(1, 50) for _ in range(512)]
    prompts = [shared + [rnd.randrange(1, 50) for _ in range(rnd.randrange(1, 120))] if i % 2 == 0 else
               [rnd.randrange(1, 50) for _ in range(rnd.randrange(200, 300))] for i in range(12)]
    params = [SamplingParams(max_tokens=rnd.randrange(20, 80), ignore_eos=True) for _ in prompts]

    def run(pipelined):
        eng = make_engine(False, 30, prefix=True)
        if pipelined:
            first = [o["tokens"] for o in eng.generate(prompts, copy.deepcopy(params), use_tqdm=False)]
        else:
            reqs = [eng.submit(p, sp) for p, sp in zip(prompts, copy.deepcopy(params))]
            while not eng.finished:
                eng.step()
            first = [r.completion_tokens for r in reqs]
        # second turn: the first turn's whole text plus a few new tokens
        turn2 = [p + c + [3, 4, 5] for p, c in zip(prompts, first)]
        reqs2 = [eng.submit(p, SamplingParams(max_tokens=5, ignore_eos=True)) for p in turn2]
        cached = []
        while not eng.finished:
            b = eng.step()
            cached += [r.num_cached_tokens for r in b.requests if b.type == Batch.PREFILL]
        return first, [r.completion_tokens for r in reqs2], cached

    plain_first, plain_second, plain_cached = run(False)
    piped_first, piped_second, piped_cached = run(True)
    assert piped_first == plain_first and piped_second == plain_second
    assert sum(plain_cached) > 0
    # the pipelined run has published (almost) the same blocks: a request may lose its last full block when
    # it finishes before that block's tokens have arrived
    assert sum(piped_cached) >= 0.8 * sum(plain_cached)


def test_prefix_cache_never_sees_placeholder_tokens():
    """A preempted request goes back to the head of the queue while its last sampled ids may still be
    placeholders on the host.  Whatever is published to the prefix cache, or counted as cached, must be
    real tokens: identical prompts in a pool so tight that requests are preempted again and again."""
    rnd = random.Random(5)
    base = [rnd.randrange(1, 50) for _ in range(250)]
    prompts = [list(base) for _ in range(8)] + [base + [rnd.randrange(1, 50) for _ in range(300)] for _ in range(4)]
    params = [SamplingParams(max_tokens=rnd.randrange(270, 330), ignore_eos=True) for _ in prompts]

    eng = make_engine(False, 9, prefix=True)
    bm = eng.scheduler.block_manager
    published, admitted = [], []
    publish, allocate = bm._publish, bm.allocate_blocks_for_prefill

    def spy_publish(bid, h, content):
        published.append(np.frombuffer(content, dtype="<i4"))
        return publish(bid, h, content)

    def spy_allocate(req):
        allocate(req)
        admitted.append((req.num_cached_tokens, list(req.tokens[:req.num_cached_tokens])))

    bm._publish, bm.allocate_blocks_for_prefill = spy_publish, spy_allocate
    preempted = []
    preempt = eng.scheduler.preempt
    eng.scheduler.preempt = lambda r: (preempted.append(r.id), preempt(r))[1]
    out = eng.generate(prompts, copy.deepcopy(params), use_tqdm=False)
    assert [len(o["tokens"]) for o in out] == [sp.max_tokens for sp in params]
    assert preempted, "the pool was not tight enough to preempt anybody"
    assert published and all((c >= 0).all() for c in published), "a block with a placeholder was published"
    assert all(min(toks, default=0) >= 0 for _, toks in admitted), "cached tokens cover a placeholder"
    assert any(n > 0 for n, _ in admitted), "no prefix-cache hit happened"

    # the block manager on its own: a prompt with an unknown id publishes nothing from that block on
    from mini_vllm_b200.engine.request import Request
    from mini_vllm_b200.kvcache.block_manager import KVCacheBlockManager
    mgr = KVCacheBlockManager(8, 256, support_prefix_cache=True)
    r = Request(list(range(1, 257)) + [5] * 255 + [-1] + [6] * 256 + [9])
    mgr.allocate_blocks_for_prefill(r)
    assert [mgr._hash[b] != -1 for b in r.blocks] == [True, False, False, False]
    r2 = Request(list(r.tokens))
    mgr.allocate_blocks_for_prefill(r2)
    assert r2.num_cached_tokens == 256
