"""End-to-end generation through the product engine (CUDA kernels, CUDA graphs, device packing)
against the oracle model driven by the same scheduler decisions: greedy token ids must agree."""
import copy
from types import SimpleNamespace

import pytest
import torch

from mini_vllm_b200.config import Config, SamplingParams, gemma3_shape, qwen3_shape
from mini_vllm_b200.engine.engine import Engine
from mini_vllm_b200.engine.request import Request
from mini_vllm_b200.scheduler.scheduler import Scheduler
from mini_vllm_b200.workloads import generator, randint
from oracle.model import OracleExecutor, OracleModel, reference_names

pytestmark = pytest.mark.gpu


def small_qwen3(**kw):
    return qwen3_shape(num_hidden_layers=2, hidden_size=256, intermediate_size=512, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=128, vocab_size=2048, max_position_embeddings=4096, **kw)


def small_gemma3(**kw):
    return gemma3_shape(num_hidden_layers=6, hidden_size=256, intermediate_size=512, num_attention_heads=4,
                        num_key_value_heads=1, head_dim=256, vocab_size=2048, max_position_embeddings=4096,
                        sliding_window=64, query_pre_attn_scalar=256, **kw)


def oracle_replay(engine: Engine, family: str, prompts, params, sched_cfg, got):
    """Teacher-forced check: the oracle model follows the product's token stream under an identical
    scheduler and scores every token the product chose.

    Returns (steps, exact, worst_deficit): the number of sampled tokens, how many equal the oracle's
    own argmax, and the largest amount by which a chosen token's oracle logit fell short of the
    oracle's maximum.  bf16 logits of magnitude ~2 carry ~1e-2 of rounding noise, so near-ties can
    flip; anything beyond a few ulps is a real error.
    """
    cfg = engine.config
    weights = reference_names({k: v.detach() for k, v in engine.executor.model.state_dict().items()},
                              family, cfg.hf_config)
    model = OracleModel(weights, cfg.hf_config, family, cfg.kv_cache_num_blocks, cfg.kv_cache_block_size,
                        device=engine.executor.device)
    ex, sch = OracleExecutor(model, cfg.kv_cache_block_size), Scheduler(sched_cfg)
    reqs = [Request(p, sp) for p, sp in zip(prompts, params)]
    index = {r.id: i for i, r in enumerate(reqs)}
    for r in reqs:
        sch.submit(r)
    steps = exact = 0
    worst = 0.0
    while not sch.finished:
        batch = sch.schedule()
        logits = ex.logits(batch).float()
        forced = [got[index[r.id]][r.num_completion_tokens] for r in batch.requests]
        chosen = logits[torch.arange(len(forced)), torch.tensor(forced, device=logits.device)]
        top = logits.max(dim=-1).values
        worst = max(worst, ((top - chosen) / top.abs().clamp_min(1.0)).max().item())
        exact += int((logits.argmax(-1).cpu() == torch.tensor(forced)).sum())
        steps += len(forced)
        sch.update(batch, forced)
    return steps, exact, worst


def check_tokens(engine, family, prompts, params, cfg, got):
    steps, exact, worst = oracle_replay(engine, family, prompts, params, cfg, got)
    assert worst <= 4 * 2 ** -8, f"a chosen token is {worst:.4f} (relative) below the oracle's best logit"
    assert exact >= 0.95 * steps, f"only {exact}/{steps} tokens equal the oracle argmax"
    return exact, steps


def small_gemma3_hf_window(**kw):
    """The same model with the Hugging Face window convention (the query counts as one of the 64 keys)."""
    return small_gemma3(sliding_window_counts_query=True, **kw)


@pytest.mark.parametrize("family,shape,graphs", [("qwen3", small_qwen3, True), ("qwen3", small_qwen3, False),
                                                  ("gemma3", small_gemma3, True),
                                                  ("gemma3", small_gemma3_hf_window, True)])
def test_greedy_tokens_match_oracle(cuda, family, shape, graphs):
    g = generator(5)
    lens = randint(g, 5, 700, 12)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in lens]
    params = [SamplingParams(max_tokens=40, ignore_eos=True) for _ in prompts]
    cfg = Config(hf_config=shape(), kv_cache_num_blocks=64, max_num_batched_seqs=8, max_num_batched_tokens=2048,
                 use_cuda_graph=graphs, gpu_memory_utilization=0.3, seed=3)
    engine = Engine(cfg)
    out = engine.generate(prompts, copy.deepcopy(params), use_tqdm=False)
    engine.executor.check_device_status()
    got = [o["tokens"] for o in out]
    assert all(len(t) == 40 for t in got)
    check_tokens(engine, family, prompts, params, cfg, got)


def test_unfused_head_matches_oracle(cuda):
    """``fused_greedy_head=False``: lm_head writes its logits and the sampler reads them, as the reference does."""
    g = generator(15)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in randint(g, 5, 500, 8)]
    params = [SamplingParams(max_tokens=24, ignore_eos=True) for _ in prompts]
    cfg = Config(hf_config=small_qwen3(), kv_cache_num_blocks=40, max_num_batched_seqs=8, max_num_batched_tokens=2048,
                 gpu_memory_utilization=0.3, seed=3, fused_greedy_head=False)
    engine = Engine(cfg)
    assert not engine.executor.fused_head
    out = engine.generate(prompts, copy.deepcopy(params), use_tqdm=False)
    check_tokens(engine, "qwen3", prompts, params, cfg, [o["tokens"] for o in out])


def test_prefix_cache_and_preemption_match_oracle(cuda):
    """A tight pool (preemptions) with the prefix cache on: shared 512-token prefixes, same tokens as the oracle."""
    g = generator(6)
    shared = torch.randint(0, 2048, (512,), generator=g).tolist()
    prompts = []
    for i in range(10):
        body = torch.randint(0, 2048, (int(torch.randint(10, 300, (1,), generator=g)),), generator=g).tolist()
        prompts.append(shared + body if i % 2 == 0 else body)
    params = [SamplingParams(max_tokens=60, ignore_eos=True) for _ in prompts]
    cfg = Config(hf_config=small_qwen3(), kv_cache_num_blocks=14, max_num_batched_seqs=6,
                 max_num_batched_tokens=4096, enable_prefix_cache=True, gpu_memory_utilization=0.3, seed=4)
    engine = Engine(cfg)
    out = engine.generate(prompts, copy.deepcopy(params), use_tqdm=False)
    engine.executor.check_device_status()
    got = [o["tokens"] for o in out]
    check_tokens(engine, "qwen3", prompts, params, cfg, got)


def test_pipelined_loop_with_preemption_matches_oracle(cuda):
    """A pool too small for everybody (requests get preempted and re-prefilled) under the pipelined step loop,
    where sampled ids reach the host late: still the oracle's tokens."""
    g = generator(7)
    prompts = [torch.randint(0, 2048, (int(n),), generator=g).tolist() for n in randint(g, 30, 500, 10)]
    params = [SamplingParams(max_tokens=150, ignore_eos=True) for _ in prompts]
    cfg = Config(hf_config=small_qwen3(), kv_cache_num_blocks=9, max_num_batched_seqs=6,
                 max_num_batched_tokens=4096, gpu_memory_utilization=0.3, seed=5)
    engine = Engine(cfg)
    assert engine._schedule_is_token_independent(params)
    out = engine.generate(prompts, copy.deepcopy(params), use_tqdm=False)
    engine.executor.check_device_status()
    got = [o["tokens"] for o in out]
    assert all(len(t) == 150 and min(t) >= 0 for t in got)
    check_tokens(engine, "qwen3", prompts, params, cfg, got)


@pytest.mark.parametrize("family,shape", [("qwen3", small_qwen3), ("gemma3", small_gemma3)])
def test_mixed_prefill_and_decode_steps_match_oracle(cuda, family, shape):
    """``enable_mixed_steps``: prompts are prefilled in the same step in which running requests decode
    (one forward pass, the prefill kernel on one part of the rows and the decode kernel on the rest).
    Few sequence slots and different output lengths, so prompts keep arriving next to decodes."""
    g = generator(12)
    prompts = [torch.randint(0, 2048, (int(n),), generator=g).tolist() for n in randint(g, 5, 600, 14)]
    params = [SamplingParams(max_tokens=int(m), ignore_eos=True) for m in randint(g, 4, 40, 14)]
    cfg = Config(hf_config=shape(), kv_cache_num_blocks=48, max_num_batched_seqs=4, max_num_batched_tokens=2048,
                 enable_mixed_steps=True, gpu_memory_utilization=0.3, seed=6)
    engine = Engine(cfg)
    kinds = []
    launch = engine.executor.launch
    def spy(batch, slots):
        kinds.append(batch.type)
        return launch(batch, slots)
    engine.executor.launch = spy
    out = engine.generate(prompts, copy.deepcopy(params), use_tqdm=False)
    got = [o["tokens"] for o in out]
    assert [len(t) for t in got] == [sp.max_tokens for sp in params]
    assert kinds.count(2) >= 3, "no mixed step was scheduled"
    check_tokens(engine, family, prompts, params, cfg, got)


def test_pipelined_loop_stops_on_eos_like_the_oracle(cuda):
    """EOS stopping under the pipelined loop: a request that emitted EOS keeps decoding until the token has
    reached the host, then is cut back.  A third of the vocabulary is EOS so that requests stop at scattered
    points; some requests ignore EOS; the pool is tight enough for preemptions."""
    g = generator(13)
    prompts = [torch.randint(0, 2048, (int(n),), generator=g).tolist() for n in randint(g, 20, 500, 16)]
    params = [SamplingParams(max_tokens=60, ignore_eos=(i % 4 == 3)) for i in range(len(prompts))]
    shape = small_qwen3()
    shape.eos_token_id = [i for i in range(2048) if i % 3 == 0]
    cfg = Config(hf_config=shape, kv_cache_num_blocks=12, max_num_batched_seqs=6, max_num_batched_tokens=4096,
                 gpu_memory_utilization=0.3, seed=9)
    assert cfg.eos_token_ids
    engine = Engine(cfg)
    assert engine._schedule_is_token_independent(params)
    out = engine.generate(prompts, copy.deepcopy(params), use_tqdm=False)
    got = [o["tokens"] for o in out]
    eos = set(cfg.eos_token_ids)
    stopped = 0
    for toks, sp in zip(got, params):
        assert 1 <= len(toks) <= 60 and min(toks) >= 0
        if sp.ignore_eos:
            assert len(toks) == 60
        else:
            assert all(t not in eos for t in toks[:-1]), "tokens were kept past an EOS"
            assert len(toks) == 60 or toks[-1] in eos
            stopped += toks[-1] in eos and len(toks) < 60
    assert stopped >= 4
    check_tokens(engine, "qwen3", prompts, params, cfg, got)


def test_sampling_params_paths(cuda):
    """Temperature alone stays greedy (reference behaviour); top-k draws are seeded and reproducible."""
    g = generator(8)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (20, 33, 65)]
    def run(sp, seed):
        cfg = Config(hf_config=small_qwen3(), kv_cache_num_blocks=16, max_num_batched_seqs=4,
                     gpu_memory_utilization=0.3, seed=seed, use_cuda_graph=False)
        return [o["tokens"] for o in Engine(cfg).generate(prompts, sp, use_tqdm=False)]
    greedy = run(SamplingParams(max_tokens=8, ignore_eos=True), 1)
    warm = run(SamplingParams(max_tokens=8, ignore_eos=True, temperature=0.5), 1)
    assert greedy == warm
    a = run(SamplingParams(max_tokens=8, ignore_eos=True, temperature=1.5, top_k=50), 1)
    b = run(SamplingParams(max_tokens=8, ignore_eos=True, temperature=1.5, top_k=50), 1)
    assert a == b and a != greedy
    k1 = run(SamplingParams(max_tokens=8, ignore_eos=True, temperature=1.5, top_k=1), 1)
    assert k1 == greedy
