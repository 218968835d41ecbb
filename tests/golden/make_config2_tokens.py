"""Make tests/golden/config2_tokens.npz: greedy token ids of the reference path on the real config-2 model shape.

Run on a machine with a B200 and the staged reference package (``python -m oracle.stage_reference``):

    python tests/golden/make_config2_tokens.py --out tests/golden/config2_tokens.npz

Model: Qwen3-0.6B shape (28 layers, hidden 1024, 16/8 heads of 128, vocabulary 151 936, tied lm_head), weights
N(0, 0.02) from seed 0, norm gains at their defaults.  Prompts: random token ids, lengths U[100, 992] (the
config-2 range, capped so that 32 tokens fit under the 1024 total).

With random weights the two largest logits of a row are about 0.13 apart on average while a bf16 logit near 3 is
spaced 0.0156, so one step in nine is an exact or near tie, and which side of a tie an implementation lands on is
rounding noise.  A 32-token greedy stream is comparable between two implementations only where no step is that
close.  So the prompt set is screened, once, here:

  1. candidates run through the product engine, recording the two largest logits of every sampled row; a candidate
     survives if all 32 steps have a margin of at least ``--min-ulps`` bf16 steps (default 2, i.e. more than one ulp);
  2. the survivors run through the REFERENCE path (the reference's scheduler, executor, packing, model and sampler,
     eager on the device, with the fp32 gather-and-SDPA standing in for its attention package); the same margin is
     required of the reference's own logits;
  3. the first ``--keep`` prompts that pass both go into the fixture with the reference's tokens and margins; the
     product engine is run once more on exactly that set, as the test will run it (its default configuration, in
     which greedy steps go through the fused lm_head + argmax kernel; the screening runs materialise logits).

Nothing is dropped for disagreeing: a prompt that passes both margin screens and still differs is kept and counted
(``mismatches_after_screen``) - it would mean the implementations are more than a rounding apart.  The first 64
unscreened config-2 prompts are also compared, as a diagnostic of what raw random prompts give.
"""
from __future__ import annotations

import argparse
import math
import sys
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))

from mini_vllm_b200.config import Config, SamplingParams, qwen3_shape  # noqa: E402
from mini_vllm_b200.engine.engine import Engine  # noqa: E402
from mini_vllm_b200.workloads import config2_requests, generator  # noqa: E402

STEPS = 32
VOCAB = 151936


def ulp_bf16(x: np.ndarray) -> np.ndarray:
    """Spacing of bf16 numbers at |x| (8 significant bits)."""
    ax = np.maximum(np.abs(x), 1e-30)
    return np.exp2(np.floor(np.log2(ax)) - 7)


def margin_ulps(top2: np.ndarray) -> np.ndarray:
    """[..., 2] (largest, second largest) -> margin in bf16 steps at the largest value."""
    return (top2[..., 0] - top2[..., 1]) / ulp_bf16(top2[..., 0])


def test_engine_config() -> Config:
    """The engine the test builds: config 2's engine settings."""
    return Config(hf_config=qwen3_shape(), kv_cache_num_blocks=512, max_num_batched_seqs=64,
                  max_num_batched_tokens=16384, gpu_memory_utilization=0.5, use_cuda_graph=True, seed=0)


def product_generate(engine: Engine, prompts):
    """Tokens and per-step (largest, second largest) logits of every request, through ``Engine.generate``.
    (The engine must materialise its logits for this: ``fused_greedy_head=False``.)"""
    ex = engine.executor
    assert not ex.fused_head, "margins can only be recorded when the logits exist"
    order, tops = [], []
    launch, sampler = ex.launch, ex.sampler

    def spy_launch(batch, slots):
        order.append([r.id for r in batch.requests])
        return launch(batch, slots)

    class SpySampler:
        def __call__(self, logits, *a, **kw):
            tops.append(torch.topk(logits, 2, dim=-1).values.float())
            return sampler(logits, *a, **kw)

    ex.launch, ex.sampler = spy_launch, SpySampler()
    try:
        out = engine.generate(prompts, SamplingParams(max_tokens=STEPS, ignore_eos=True), use_tqdm=False)
    finally:
        ex.launch, ex.sampler = launch, sampler
    # request ids grow with submission order inside this call
    first_id = min(i for ids in order for i in ids)
    per_req = [[] for _ in prompts]
    for ids, t in zip(order, tops):
        for rid, pair in zip(ids, t.cpu().tolist()):
            per_req[rid - first_id].append(pair)
    assert all(len(p) == STEPS for p in per_req), "a request was preempted or cut: enlarge the pool"
    return [o["tokens"] for o in out], np.asarray(per_req, dtype=np.float32)


def candidate_prompts(g: torch.Generator, n: int):
    lens = torch.randint(100, 993, (n,), generator=g).tolist()
    return [torch.randint(0, VOCAB, (m,), generator=g).tolist() for m in lens]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=str(ROOT / "tests" / "golden" / "config2_tokens.npz"))
    ap.add_argument("--keep", type=int, default=16)
    ap.add_argument("--chunk", type=int, default=2048)
    ap.add_argument("--max-candidates", type=int, default=65536)
    ap.add_argument("--min-ulps", type=float, default=2.0)
    ap.add_argument("--seed", type=int, default=2)
    ap.add_argument("--reference", default="auto", choices=["auto", "engine", "port"],
                    help="engine: the staged reference package; port: oracle.model.OracleModel; auto: engine if staged")
    args = ap.parse_args()

    from oracle import reference_engine
    from oracle.model import OracleExecutor, OracleModel, reference_names
    use_engine = args.reference == "engine" or (args.reference == "auto" and reference_engine.available())
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)

    # ---- the big engine for screening -------------------------------------------------------------------
    big = Engine(Config(hf_config=qwen3_shape(), kv_cache_num_blocks=4 * 512 + 64, max_num_batched_seqs=512,
                        max_graph_batch_size=512, max_num_batched_tokens=16384, gpu_memory_utilization=0.6,
                        use_cuda_graph=True, seed=0, fused_greedy_head=False))
    weights = reference_names({k: v.detach() for k, v in big.executor.model.state_dict().items()}, "qwen3",
                              big.config.hf_config)

    if use_engine:
        ref = reference_engine.ReferenceEngine(big.config.hf_config, weights, dev, kv_cache_num_blocks=4 * 64 + 8,
                                               max_num_batched_seqs=64)
        ref_kind = "reference engine (staged package, eager, fp32 gather-and-SDPA attention)"

        def reference_generate(prompts):
            toks, top2 = ref.generate(prompts, STEPS)
            return toks, np.asarray(top2, dtype=np.float32)
    else:
        ref_kind = "oracle port (oracle.model.OracleModel on the device)"
        from mini_vllm_b200.engine.request import Request
        from mini_vllm_b200.scheduler.scheduler import Scheduler
        cfg = Config(hf_config=qwen3_shape(), kv_cache_num_blocks=4 * 64 + 8, max_num_batched_seqs=64, seed=0)
        omodel = OracleModel(weights, cfg.hf_config, "qwen3", cfg.kv_cache_num_blocks, 256, device=dev)

        def reference_generate(prompts):
            ex, sch = OracleExecutor(omodel, 256), Scheduler(cfg)
            reqs = [Request(p, SamplingParams(max_tokens=STEPS, ignore_eos=True)) for p in prompts]
            top2 = {r.id: [] for r in reqs}
            for r in reqs:
                sch.submit(r)
            while not sch.finished:
                batch = sch.schedule()
                logits = ex.logits(batch)
                for r, pair in zip(batch.requests, torch.topk(logits.float(), 2, dim=-1).values.cpu().tolist()):
                    top2[r.id].append(pair)
                sch.update(batch, torch.argmax(logits, dim=-1).tolist())
            return [r.completion_tokens for r in reqs], np.asarray([top2[r.id] for r in reqs], dtype=np.float32)

    # ---- diagnostic: the first 64 config-2 prompts, unscreened ----------------------------------------------
    raw = [r.prompt[:992] for r in config2_requests(seed=0, n=64)]
    t0 = time.time()
    raw_prod, raw_prod_top2 = product_generate(big, raw)
    raw_ref, raw_ref_top2 = reference_generate(raw)
    raw_same = [p == r for p, r in zip(raw_prod, raw_ref)]
    raw_first_diff = [next((i for i, (a, b) in enumerate(zip(p, r)) if a != b), STEPS) for p, r in zip(raw_prod, raw_ref)]
    raw_ref_m = margin_ulps(raw_ref_top2)
    raw_margin_at_diff = [float(raw_ref_m[i, s]) if s < STEPS else math.nan for i, s in enumerate(raw_first_diff)]
    print(f"unscreened: {sum(raw_same)}/64 prompts identical over {STEPS} tokens; reference margin (bf16 steps) at the "
          f"first difference: {sorted(round(m, 2) for m in raw_margin_at_diff if not math.isnan(m))}  "
          f"[{time.time() - t0:.0f} s]", flush=True)
    steps_tied = float((raw_ref_m < 1.0).mean())
    print(f"unscreened: {steps_tied:.3f} of reference steps have a margin under one bf16 step", flush=True)

    # ---- screening -----------------------------------------------------------------------------------------
    g = generator(args.seed)
    kept_prompts, kept_ref_tokens, kept_ref_top2 = [], [], []
    n_cand = n_stage1 = n_stage2 = mismatches = 0
    while len(kept_prompts) < args.keep and n_cand < args.max_candidates:
        cands = candidate_prompts(g, args.chunk)
        n_cand += len(cands)
        toks, top2 = product_generate(big, cands)
        ok = margin_ulps(top2).min(axis=1) >= args.min_ulps
        survivors = [i for i in range(len(cands)) if ok[i]]
        n_stage1 += len(survivors)
        if survivors:
            sp = [cands[i] for i in survivors]
            rt, rtop2 = reference_generate(sp)
            rok = margin_ulps(rtop2).min(axis=1) >= args.min_ulps
            for j, i in enumerate(survivors):
                if not rok[j]:
                    continue
                n_stage2 += 1
                if rt[j] != toks[i]:
                    mismatches += 1
                if len(kept_prompts) < args.keep:
                    kept_prompts.append(cands[i]); kept_ref_tokens.append(rt[j]); kept_ref_top2.append(rtop2[j])
        print(f"candidates {n_cand}: {n_stage1} pass the product margin, {n_stage2} also the reference margin, "
              f"{mismatches} of those differ  [{time.time() - t0:.0f} s]", flush=True)
    if not kept_prompts:
        sys.exit("no prompt passed the screen")

    # ---- the kept set through the engine the test will build ------------------------------------------------
    del big
    torch.cuda.empty_cache()
    small = Engine(test_engine_config())                       # the default engine: fused lm_head + argmax, no logits
    out = small.generate(kept_prompts, SamplingParams(max_tokens=STEPS, ignore_eos=True), use_tqdm=False)
    final_tokens = [o["tokens"] for o in out]
    same = [a == b for a, b in zip(final_tokens, kept_ref_tokens)]
    print(f"kept set: {sum(same)}/{len(same)} identical to the reference over {STEPS} tokens", flush=True)

    lens = np.asarray([len(p) for p in kept_prompts], np.int32)
    np.savez_compressed(
        args.out, prompt_lens=lens, prompts_flat=np.concatenate([np.asarray(p, np.int32) for p in kept_prompts]),
        ref_tokens=np.asarray(kept_ref_tokens, np.int32), ref_top2=np.asarray(kept_ref_top2, np.float32),
        ref_margin_ulps=margin_ulps(np.asarray(kept_ref_top2, np.float32)).astype(np.float32),
        product_tokens=np.asarray(final_tokens, np.int32),
        reference_kind=np.asarray(ref_kind), seed=np.asarray(args.seed), min_ulps=np.asarray(args.min_ulps),
        candidates=np.asarray(n_cand), pass_product_margin=np.asarray(n_stage1), pass_both_margins=np.asarray(n_stage2),
        mismatches_after_screen=np.asarray(mismatches),
        unscreened_identical=np.asarray(sum(raw_same)), unscreened_first_diff=np.asarray(raw_first_diff, np.int32),
        unscreened_ref_margin_at_diff=np.asarray(raw_margin_at_diff, np.float32),
        unscreened_steps_under_one_ulp=np.asarray(steps_tied))
    print(f"wrote {args.out}: {len(kept_prompts)} prompts from {n_cand} candidates ({ref_kind})")


if __name__ == "__main__":
    main()
