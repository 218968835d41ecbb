"""The reference's own scheduler / executor / model code, stepped like its Engine, against the oracle restatement.

The reference package is imported from the staged copy (``oracle/stage_reference.py``); where neither the staged
copy nor a checkout next to this repository exists the test is skipped.  On a host without a GPU the runner swaps in
the restated KV write for the Triton kernel; everything else (packing, block ids, batch order, model wiring, argmax
sampler) is the reference's.  The oracle executor under the product's scheduler must produce the same greedy tokens,
which pins the whole CPU baseline loop of ``bench.py`` - scheduler, packing, model, sampler - to the reference.
"""
import copy

import pytest
import torch

from mini_vllm_b200.config import Config, SamplingParams, qwen3_shape
from mini_vllm_b200.engine.request import Request
from mini_vllm_b200.models.loader import load_model
from mini_vllm_b200.scheduler.scheduler import Scheduler
from mini_vllm_b200.workloads import generator, randint
from oracle import reference_engine, stage_reference
from oracle.model import OracleExecutor, OracleModel, reference_names


@pytest.fixture(scope="module")
def staged():
    if stage_reference.stage() is None:
        pytest.skip("no reference checkout and no staged copy")


def test_reference_engine_loop_matches_the_oracle_executor(staged):
    hf = qwen3_shape(num_hidden_layers=2, hidden_size=128, intermediate_size=256, num_attention_heads=4,
                     num_key_value_heads=2, head_dim=32, vocab_size=499, max_position_embeddings=2048)
    cfg = Config(hf_config=hf, kv_cache_num_blocks=12, max_num_batched_seqs=4, max_num_batched_tokens=1024,
                 use_cuda_graph=False, seed=11)
    model = load_model(cfg, device="cpu")
    weights = reference_names({k: v.detach() for k, v in model.state_dict().items()}, "qwen3", hf)
    g = generator(21)
    prompts = [torch.randint(0, 499, (n,), generator=g).tolist() for n in randint(g, 3, 400, 9)]
    steps = 12

    ref = reference_engine.ReferenceEngine(hf, weights, "cpu", kv_cache_num_blocks=12, max_num_batched_seqs=4,
                                           max_num_batched_tokens=1024)
    ref_tokens, ref_top2 = ref.generate(prompts, steps)
    assert all(len(t) == steps and len(m) == steps for t, m in zip(ref_tokens, ref_top2))

    ex = OracleExecutor(OracleModel(weights, hf, "qwen3", 12, 256), 256)
    sch = Scheduler(cfg)
    reqs = [Request(p, SamplingParams(max_tokens=steps, ignore_eos=True)) for p in prompts]
    for r in reqs:
        sch.submit(r)
    while not sch.finished:
        batch = sch.schedule()
        sch.update(batch, ex.execute(batch))
    got = [r.completion_tokens for r in reqs]

    # same machine, same eager arithmetic: the streams agree wherever the reference's own margin is not a tie
    for toks, want, pairs in zip(got, ref_tokens, ref_top2):
        for i, (a, b) in enumerate(zip(toks, want)):
            if a != b:
                assert pairs[i][0] == pairs[i][1], f"token {i}: {a} vs {b} with margin {pairs[i]}"
                break
    same = sum(t == w for t, w in zip(got, ref_tokens))
    assert same >= len(prompts) - 1
