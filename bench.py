#!/usr/bin/env python
"""Benchmark of the ragged continuous-batching attention path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Workload (``config.workload``): Qwen3-0.6B-shape random-init model, greedy decoding, continuous batching.
Default: the per-GPU share of the box-scale offline-serving job the headline metric is quoted on
(4096 requests over 8 GPUs = 512 requests per GPU, prompt lengths log-uniform [32,4096], output lengths
U[64,1024], random token ids); ``--workload config2`` selects the 64-request job (prompt U[100,1024],
prompt+output <= 1024).  One "step" is one complete generation job over the rank's request set.  At
N > 1 each rank is an independent engine replica (no collective on the data path); the global list of
512*N requests is partitioned by the host dispatcher by token count, so per-GPU work is fixed (weak
scaling) and N = 8 is exactly the 4096-request job.

Metric: prompt+generated tokens per second, whole job, all GPUs.
* ``value``: the job's device time, CUDA events around its first and last kernel (the engine's step loop
  is pipelined: sampled ids stay in HBM and feed the next step's packing kernel).
* ``e2e``: the same job through ``Engine.generate`` with host token lists in and out (wall clock:
  request submission, every step's metadata upload, every step's token read-back and the final list
  assembly are inside the timed region).
* ``roofline``: decode attention kernel, the largest kernel of the step: K/V bytes of the contexts
  it read / CUDA-event time, replayed on contexts recorded during the job, against the measured
  HBM copy bandwidth.  ``kernels`` adds the same figure on the fixed 240-sequence decode batch
  (contexts U[128,4096]) and the prefill kernel's TFLOP/s.
* ``cpu_baseline`` / ``--impl reference``: the oracle restatement of the reference's PyTorch path
  timed on the host cores on a bounded sample of the same workload (per-token extrapolation).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from mini_vllm_b200.config import Config, SamplingParams, qwen3_shape  # noqa: E402
from mini_vllm_b200.dispatcher import partition_by_tokens, request_cost  # noqa: E402
from mini_vllm_b200.workloads import (GEMMA3_1B, QWEN3_0P6B, config2_requests, config3, config4,  # noqa: E402
                                       decode_kv_bytes, prefill_flops)

METRIC = "ragged prefill+decode tokens/s (Qwen3-0.6B shapes, continuous batching, greedy)"
WORKLOADS = {
    "config5": "config5 share: Qwen3-0.6B random-init, 512 req/GPU (one of the 8 shares of 4096 requests per GPU), "
               "prompt log-U[32,4096], output U[64,1024], continuous batching",
    "config2": "config2: Qwen3-0.6B random-init, 64 req/GPU, prompt U[100,1024], total<=1024, continuous batching",
}


def workload_requests(workload: str, world: int = 1, rank: int = 0):
    """The requests of one replica.

    Requests are split by token count - the K/V tokens a request will have read by its end, one context per
    generated token: out * (prompt + out / 2).  (The plain prompt + output sum balances the token totals to
    0.01 % but leaves the replicas' attention work 3 % apart, and a job is bound by its slowest replica.)
    Config 5 is 4096 requests over 8 GPUs: it is cut into its 8 shares once, and a run on N GPUs takes the
    first N of them, so every replica's job is the same at every N."""
    kv_tokens = lambda r: request_cost(len(r.prompt), r.max_tokens)
    if workload == "config5" and world <= 8:
        from mini_vllm_b200.workloads import config5_requests
        all_reqs, parts = config5_requests(seed=0, n=4096), 8
    elif workload == "config5":
        from mini_vllm_b200.workloads import config5_requests
        all_reqs, parts = config5_requests(seed=0, n=512 * world), world
    else:
        all_reqs, parts = config2_requests(seed=0, n=64 * world), world
    return [all_reqs[i] for i in partition_by_tokens([kv_tokens(r) for r in all_reqs], parts)[rank]]


def measured_peaks() -> tuple[dict, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return json.loads(p.read_text()), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc = gpu_index, None
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        rows = [r.split(", ") for r in Path(self.file.name).read_text().strip().splitlines() if r.count(",") >= 8]
        os.unlink(self.file.name)
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = [float(r[1]) for r in rows]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in rows for n, v in zip(names, r[5:9]) if v.strip().lower().startswith("active")})
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": float(rows[0][2]), "samples": len(rows),
                "power_w_max": max(float(r[3]) for r in rows), "reasons": reasons}


# ---------------------------------------------------------------------------------------------------
def build_config(workload: str = "config5") -> Config:
    if workload == "config5":        # long prompts, hundreds of live sequences: a large pool, preemption allowed
        # up to 512 live sequences (the reference's default max_num_batched_seqs), all decode batches from graphs
        return Config(hf_config=qwen3_shape(), kv_cache_num_blocks=4096,
                      max_num_batched_seqs=512, max_graph_batch_size=512,
                      max_num_batched_tokens=16384, gpu_memory_utilization=0.85, use_cuda_graph=True, seed=0)
    return Config(hf_config=qwen3_shape(), kv_cache_num_blocks=512, max_num_batched_seqs=64,
                  max_num_batched_tokens=16384, gpu_memory_utilization=0.5, use_cuda_graph=True, seed=0)


def build_engine(local_rank: int, workload: str = "config5", mixed_steps: bool = False, fused_head: bool = True):
    import dataclasses
    from mini_vllm_b200.engine.engine import Engine
    torch.cuda.set_device(local_rank)
    return Engine(dataclasses.replace(build_config(workload), enable_mixed_steps=mixed_steps, fused_greedy_head=fused_head))


class ContextSpy:
    """Records the contexts of every 40th decode step of a job (for the in-situ roofline replay)."""

    def __init__(self, executor, sink):
        self.ex, self.sink, self.count, self.orig = executor, sink, 0, executor.launch

    def __enter__(self):
        if self.sink is not None:
            def spy(batch, slots):
                if batch.type == 1:
                    if self.count % 40 == 20:
                        self.sink.append(([len(r.tokens) for r in batch.requests], [list(r.blocks) for r in batch.requests]))
                    self.count += 1
                return self.orig(batch, slots)
            self.ex.launch = spy
        return self

    def __exit__(self, *exc):
        self.ex.launch = self.orig
        return False


def run_job(engine, reqs, record_contexts=None, group=None):
    """One generation job through the public API; returns (tokens processed, wall seconds, this rank's cuda ms).

    ``group is None``: this process's ``Engine.generate`` on ``reqs``.  Otherwise a collective over the ranks of
    ``group``: rank 0 holds ``reqs`` (ALL requests of the job), the host dispatcher scatters the shares, every rank
    generates, rank 0 gathers and merges; the wall time on rank 0 covers all of it and the token count is taken from
    the merged results (other ranks return 0 tokens).
    """
    prompts = params = None
    if reqs is not None:
        prompts = [r.prompt for r in reqs]
        params = [SamplingParams(max_tokens=r.max_tokens, ignore_eos=True) for r in reqs]
    torch.cuda.synchronize()
    with ContextSpy(engine.executor, record_contexts):
        t0 = time.perf_counter()
        if group is None:
            out = engine.generate(prompts, params, use_tqdm=False)
        else:
            from mini_vllm_b200.dispatcher import generate_over_ranks
            out = generate_over_ranks(engine, prompts, params, group=group)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
    n_tok = 0
    if out is not None:
        n_tok = sum(len(p) for p in prompts) + sum(len(o["tokens"]) for o in out)
        assert all(len(o["tokens"]) == r.max_tokens for o, r in zip(out, reqs))
    return n_tok, wall, engine.last_job_device_ms


def decode_roofline(engine, contexts, peaks):
    """Replay the decode-attention kernel on recorded step contexts over the engine's own KV pool."""
    from mini_vllm_b200 import ops
    from mini_vllm_b200.workloads import table_tensor
    ex = engine.executor
    dev, hf = ex.device, engine.config.hf_config
    hq, hkv, d, layers = hf.num_attention_heads, hf.num_key_value_heads, hf.head_dim, hf.num_hidden_layers
    total_bytes = total_ms = 0.0
    launches = 0
    for lens, blocks in contexts:
        b = len(lens)
        q = torch.randn(b, hq, d, device=dev, dtype=torch.bfloat16)
        seqlens = torch.tensor(lens, dtype=torch.int32, device=dev)
        bt = table_tensor(blocks).to(dev)
        ws = ops.decode_workspace(b, hq, d, dev)
        out = torch.empty_like(q)
        ops.decode_plan(seqlens, -1, hq, hkv, d, ws, block_table=bt, block_size=256)
        def all_layers():                                        # distinct layer pools: no L2 reuse between launches
            for layer in range(layers):
                ops.decode_attn(q, ex.kv_cache[0, layer], ex.kv_cache[1, layer], seqlens, bt, d ** -0.5, -1, ws, out=out)
        all_layers()                                             # warm-up, also outside any capture
        torch.cuda.synchronize()
        # launch the 28 layers back to back from a CUDA graph, as the engine does, so that the
        # event-to-event time is device time and not the host's launch rate
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            all_layers()
        graph.replay()
        reps = 3
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        total_ms += e0.elapsed_time(e1) / reps
        total_bytes += layers * decode_kv_bytes(QWEN3_0P6B, lens)
        launches += layers
    achieved = total_bytes / (total_ms * 1e-3) / 1e9 if total_ms else 0.0
    return {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": round(achieved / peaks["hbm_gbs"], 4),
            # ncu on the 2.063 GB config-3 launch read 2.0733 GB and wrote 5.8 MB (profiles/): traffic is
            # 1.008 x the algorithmic bytes and grows in proportion, so it is scaled to this launch size
            "traffic": int(1.008 * total_bytes / max(launches, 1)), "kernel": "decode_attn_kernel<128,8>",
            "launches_timed": launches, "avg_launch_us": round(total_ms * 1e3 / max(launches, 1), 2),
            "avg_bytes_per_launch": int(total_bytes / max(launches, 1)),
            "note": "algorithmic K+V bytes of recorded decode steps, 28 layer launches replayed from a CUDA graph; peak = STREAM copy"}


LEGS = ("attn3", "prefill", "attn4", "sampler", "rope", "pack", "head", "glue")


def graph_time_ms(sweep, launches_per_sweep: int, reps: int = 5) -> float:
    """Device time per launch of ``sweep`` (a function that enqueues ``launches_per_sweep`` kernels over
    distinct buffers), replayed from a CUDA graph so that short kernels are not timed at the host's launch rate."""
    sweep()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        sweep()
    graph.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (reps * launches_per_sweep)


def rope_and_pack_legs(dev, peaks, legs) -> dict:
    """The elementwise and integer kernels of the path on config-3 / config-5 sized steps."""
    from mini_vllm_b200 import ops
    from mini_vllm_b200.models.layers.rotary import build_cos_sin_cache
    import numpy as np
    out = {}
    hq, hkv, d = 16, 8, 128
    case, g = config3()
    q_lens = [n - c for n, c in zip(case.prefill_lens, case.prefill_cached)]
    if "rope" in legs:
        table = build_cos_sin_cache(d, 8192, 1e6).to(dev)
        wq = torch.ones(d, device=dev, dtype=torch.bfloat16)
        for name, tokens in (("prefill12784", sum(q_lens)), ("decode512", 512)):
            nbuf = max(2, min(8, int(400e6 / (tokens * (hq + 2 * hkv) * d * 2))))
            qkvs = [torch.randn(tokens, (hq + 2 * hkv) * d, device=dev).to(torch.bfloat16) for _ in range(nbuf)]
            pools = [torch.zeros(2, tokens // 256 + 2, 256, hkv, d, device=dev, dtype=torch.bfloat16) for _ in range(nbuf)]
            pos = torch.arange(tokens, device=dev, dtype=torch.int64) % 4096
            slots = torch.randperm(tokens, device=dev).to(torch.int32)          # every token its own slot, scattered
            views = [tuple(t.view(tokens, -1, d) for t in x.split([hq * d, hkv * d, hkv * d], dim=-1)) for x in qkvs]
            # q, k, v read where the projection left them; q written back in place, k and v to their cache slots
            byts = tokens * (hq + 2 * hkv) * d * 2 * 2
            for kern, call in (("rope_kv_write", lambda v3, p: ops.rope_kv_write(v3[0], v3[1], v3[2], pos, table, slots, p[0], p[1], k_in_place=False)),
                               ("qk_norm_rope_kv_write", lambda v3, p: ops.qk_norm_rope_kv_write(v3[0], v3[1], v3[2], wq, wq, 1e-6, False, pos, table, slots, p[0], p[1], k_in_place=False))):
                ms = graph_time_ms(lambda: [call(v3, p) for v3, p in zip(views, pools)], nbuf)
                out[f"{kern}_{name}"] = {"GB/s": round(byts / ms / 1e6, 1), "us": round(ms * 1e3, 2), "bytes": byts,
                                         "frac_of_measured_hbm": round(byts / ms / 1e6 / peaks["hbm_gbs"], 4)}
            del qkvs, pools, views
    if "glue" in legs:
        # the decoder glue between the GEMMs on config 3's prefill rows (Qwen3-0.6B: hidden 1024, intermediate 3072)
        hidden, inter = 1024, 3072
        for name, tokens in (("prefill12784", sum(q_lens)), ("decode512", 512)):
            nbuf = max(2, min(8, int(400e6 / (tokens * inter * 6))))
            gus = [torch.randn(tokens, 2 * inter, device=dev).to(torch.bfloat16) for _ in range(nbuf)]
            outs = [torch.empty(tokens, inter, device=dev, dtype=torch.bfloat16) for _ in range(nbuf)]
            byts = tokens * inter * 2 * 3
            ms = graph_time_ms(lambda: [ops.act_mul(gu, inter, False, out=o) for gu, o in zip(gus, outs)], nbuf)
            out[f"act_mul_{name}"] = {"GB/s": round(byts / ms / 1e6, 1), "us": round(ms * 1e3, 2), "bytes": byts,
                                      "frac_of_measured_hbm": round(byts / ms / 1e6 / peaks["hbm_gbs"], 4)}
            del gus, outs
            nbuf = 8
            xs = [torch.randn(tokens, hidden, device=dev).to(torch.bfloat16) for _ in range(nbuf)]
            ys = [torch.randn(tokens, hidden, device=dev).to(torch.bfloat16) for _ in range(nbuf)]
            os_ = [torch.empty(tokens, hidden, device=dev, dtype=torch.bfloat16) for _ in range(nbuf)]
            w = torch.ones(hidden, device=dev, dtype=torch.bfloat16)
            byts = tokens * hidden * 2 * 4                     # x and y read, x and the normed row written
            ms = graph_time_ms(lambda: [ops.add_rmsnorm(x, y, w, 1e-6, False, out=o) for x, y, o in zip(xs, ys, os_)], nbuf)
            out[f"add_rmsnorm_{name}"] = {"GB/s": round(byts / ms / 1e6, 1), "us": round(ms * 1e3, 2), "bytes": byts,
                                          "frac_of_measured_hbm": round(byts / ms / 1e6 / peaks["hbm_gbs"], 4)}
            del xs, ys, os_
    if "pack" in legs:
        # prefill packing of config 3's 16 prompts (12 784 new tokens, cached prefixes) and decode packing of 512 rows
        seq_len = np.asarray(case.prefill_lens, np.int32)
        cached = np.asarray(case.prefill_cached, np.int32)
        nblk = np.asarray([len(b) for b in case.prefill_blocks], np.int32)
        blk_off = np.concatenate([[0], np.cumsum(nblk)]).astype(np.int32)
        blocks = np.concatenate([np.asarray(b, np.int32) for b in case.prefill_blocks])
        t = int((seq_len - cached).sum())
        toks = torch.randint(0, 151936, (t,), generator=g).numpy().astype(np.int32)
        meta = torch.from_numpy(np.concatenate([seq_len, cached, blk_off, blocks, toks])).to(dev)
        ms = graph_time_ms(lambda: [ops.pack_prefill(meta, 16, t, int(blk_off[-1]), int(nblk.max()), 256, True) for _ in range(8)], 8)
        out["pack_prefill_config3"] = {"us": round(ms * 1e3, 2), "tokens": t, "out_bytes": t * 20 + 16 * int(nblk.max()) * 4}
        b = 512
        ctx = torch.randint(32, 5120, (b,), generator=g).numpy().astype(np.int32)
        nb = (ctx + 255) // 256
        off = np.concatenate([[0], np.cumsum(nb)]).astype(np.int32)
        flat = np.arange(int(off[-1]), dtype=np.int32)
        meta = torch.from_numpy(np.concatenate([ctx, off, flat, np.zeros(b, np.int32), np.full(b, -1, np.int32)])).to(dev)
        ids, pos = torch.empty(b, dtype=torch.int64, device=dev), torch.empty(b, dtype=torch.int64, device=dev)
        slot, lens = torch.empty(b, dtype=torch.int32, device=dev), torch.empty(b, dtype=torch.int32, device=dev)
        table = torch.empty(b, 4096, dtype=torch.int32, device=dev)[:, :int(nb.max())]   # row stride of a graph runner's table
        ms = graph_time_ms(lambda: [ops.pack_decode(meta, b, int(off[-1]), int(nb.max()), 256, ids, pos, slot, lens, table)
                                    for _ in range(8)], 8)
        out["pack_decode_512"] = {"us": round(ms * 1e3, 2), "rows": b, "out_bytes": b * (8 + 8 + 4 + 4 + int(nb.max()) * 4)}
    return out


def head_legs(dev, peaks) -> dict:
    """lm_head + greedy sampling on Qwen3's head (hidden 1024, vocabulary 151 936): the fused kernel against the
    cuBLAS GEMM followed by the greedy sampler.  The floor of either is reading the 311 MB weight matrix once."""
    from mini_vllm_b200 import ops
    out = {}
    hidden, vocab = 1024, 151936
    ws = [(torch.randn(vocab, hidden, device=dev) * 0.02).to(torch.bfloat16) for _ in range(2)]   # 2 x 311 MB > L2
    for rows in (512, 256, 128, 64):
        xs = [torch.randn(rows, hidden, device=dev).to(torch.bfloat16) for _ in range(2)]
        scratch = ops.lm_head_argmax_scratch(rows, dev)
        tok = torch.empty(rows, dtype=torch.int64, device=dev)
        logits = torch.empty(rows, vocab, dtype=torch.bfloat16, device=dev)
        flops, w_bytes = 2 * rows * hidden * vocab, vocab * hidden * 2

        def unfused():
            for x, w in zip(xs, ws):
                torch.matmul(x, w.t(), out=logits)
                ops.sample(logits, out=tok)
        ms_fused = graph_time_ms(lambda: [ops.lm_head_argmax(x, w, scratch, out=tok) for x, w in zip(xs, ws)], 2)
        ms_unfused = graph_time_ms(unfused, 2)
        out[f"lm_head_argmax_{rows}"] = {"us": round(ms_fused * 1e3, 1), "unfused_us": round(ms_unfused * 1e3, 1),
                                         "TFLOP/s": round(flops / ms_fused / 1e9, 1),
                                         "weight_GB/s": round(w_bytes / ms_fused / 1e6, 1),
                                         "frac_of_measured_bf16": round(flops / ms_fused / 1e9 / peaks["bf16_tflops"], 4),
                                         "frac_of_measured_hbm": round(w_bytes / ms_fused / 1e6 / peaks["hbm_gbs"], 4)}
    return out


def kernel_extras(dev, peaks, nl=4, legs=LEGS):
    """Fixed single-layer cases: the 240-sequence decode batch and the 16-sequence prefill batch.

    ``nl`` distinct KV pools (2.3 GB each) are rotated so that consecutive launches share nothing in L2.
    """
    out = {}
    if "attn3" in legs or "prefill" in legs:
        out.update(attention_legs_qwen3(dev, peaks, nl, legs))
    if "attn4" in legs:
        out.update(decode_legs_gemma3(dev, peaks, nl))
    if "sampler" in legs:
        out.update(sampler_legs(dev, peaks))
    out.update(rope_and_pack_legs(dev, peaks, legs))
    if "head" in legs:
        out.update(head_legs(dev, peaks))
    return out


def decode_leg_config3(dev, peaks, nl, case, pools, out):
    from mini_vllm_b200 import ops
    from mini_vllm_b200.workloads import table_tensor
    hq, hkv, d = 16, 8, 128
    # decode part
    b = len(case.decode_ctx)
    q = torch.randn(b, hq, d, device=dev, dtype=torch.bfloat16)
    lens = torch.tensor(case.decode_ctx, dtype=torch.int32, device=dev)
    bt = table_tensor(case.decode_blocks).to(dev)
    ws = ops.decode_workspace(b, hq, d, dev)
    o = torch.empty_like(q)
    ops.decode_plan(lens, -1, hq, hkv, d, ws, block_table=bt, block_size=256)
    ms = event_time_ms(lambda i: ops.decode_attn(q, pools[i % nl][0], pools[i % nl][1], lens, bt, d ** -0.5, -1, ws, out=o),
                       24, warm=8)
    byts = decode_kv_bytes(QWEN3_0P6B, case.decode_ctx)
    gbs = byts / ms / 1e6
    out["decode_attn_config3"] = {"GB/s": round(gbs, 1), "us": round(ms * 1e3, 1), "bytes": byts,
                                  "frac_of_measured_hbm": round(gbs / peaks["hbm_gbs"], 4),
                                  "frac_of_8TBs_nominal": round(gbs / 8000.0, 4)}
    return out


def event_time_ms(call, iters: int, warm: int = 3) -> float:
    """Median device time of ``call(i)`` over ``iters`` launches, CUDA events on the launching stream."""
    for i in range(warm):
        call(i)
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(iters + 1)]
    evs[0].record()
    for i in range(iters):
        call(i)
        evs[i + 1].record()
    torch.cuda.synchronize()
    return statistics.median(evs[i].elapsed_time(evs[i + 1]) for i in range(iters))


def attention_legs_qwen3(dev, peaks, nl, legs):
    from mini_vllm_b200 import ops
    from mini_vllm_b200.workloads import table_tensor
    case, _ = config3()
    hq, hkv, d = 16, 8, 128
    pools = [torch.randn(2, case.pool_blocks, 256, hkv, d, device=dev, dtype=torch.bfloat16) for _ in range(nl)]
    out = {}
    if "attn3" in legs:
        decode_leg_config3(dev, peaks, nl, case, pools, out)
    if "prefill" not in legs:
        return out
    cu = lambda xs: torch.tensor([0] + list(torch.tensor(xs).cumsum(0)), dtype=torch.int32, device=dev)
    # prefill part (paged, half the sequences with a cached 512-token prefix)
    q_lens = [n - c for n, c in zip(case.prefill_lens, case.prefill_cached)]
    qp = torch.randn(sum(q_lens), hq, d, device=dev, dtype=torch.bfloat16)
    btp = table_tensor(case.prefill_blocks).to(dev)
    cq, ck = cu(q_lens), cu(case.prefill_lens)
    # the launch's work list, built on the host from the lengths as the executor does while packing the step
    rows = ops.prefill_item_rows(hq, hkv, d)
    work = lambda ql, kl: torch.from_numpy(ops.build_prefill_items(ql, kl, rows)).to(dev)
    items = work(q_lens, case.prefill_lens)
    fl = prefill_flops(QWEN3_0P6B, case.prefill_lens, case.prefill_cached)
    for name, it in (("prefill_attn_config3", items), ("prefill_attn_config3_no_list", None)):
        ms = event_time_ms(lambda i: ops.prefill_attn(qp, pools[i % nl][0], pools[i % nl][1], cq, ck, max(q_lens), d ** -0.5,
                                                      -1, block_table=btp, items=it), 10)
        tf = fl / ms / 1e9
        out[name] = {"TFLOP/s": round(tf, 1), "us": round(ms * 1e3, 1), "flops": fl,
                     "frac_of_measured_bf16": round(tf / peaks["bf16_tflops"], 4)}
    del pools
    # the same kernel on long and on short prompts (dense K/V): 4 x 8192 and 32 x 1024 tokens
    for name, (nseq, slen) in (("prefill_attn_4x8192", (4, 8192)), ("prefill_attn_32x1024", (32, 1024))):
        lens_p = [slen] * nseq
        qd = torch.randn(nseq * slen, hq, d, device=dev, dtype=torch.bfloat16)
        kd = torch.randn(nseq * slen, hkv, d, device=dev, dtype=torch.bfloat16)
        vd = torch.randn(nseq * slen, hkv, d, device=dev, dtype=torch.bfloat16)
        cd = cu(lens_p)
        fl = prefill_flops(QWEN3_0P6B, lens_p, [0] * nseq)
        for key, it in ((name, work(lens_p, lens_p)), (name + "_no_list", None)):
            ms = event_time_ms(lambda i: ops.prefill_attn(qd, kd, vd, cd, cd, slen, d ** -0.5, -1, items=it), 10)
            out[key] = {"TFLOP/s": round(fl / ms / 1e9, 1), "us": round(ms * 1e3, 1), "flops": fl,
                        "frac_of_measured_bf16": round(fl / ms / 1e9 / peaks["bf16_tflops"], 4)}
        del qd, kd, vd
    return out


def decode_legs_gemma3(dev, peaks, nl):
    """Gemma3-1B shapes (4 q heads, 1 kv head, head_dim 256), 128 sequences, contexts U[512,4096]: a global layer
    and a sliding-window-512 layer (window layers count only the visible keys)."""
    from mini_vllm_b200 import ops
    from mini_vllm_b200.workloads import table_tensor
    out = {}
    g4, _ = config4()
    hq, hkv, d = 4, 1, 256
    gpools = [torch.randn(2, g4.pool_blocks, 256, hkv, d, device=dev, dtype=torch.bfloat16) for _ in range(max(nl, 2) * 2)]
    b = len(g4.decode_ctx)
    q = torch.randn(b, hq, d, device=dev, dtype=torch.bfloat16)
    lens = torch.tensor(g4.decode_ctx, dtype=torch.int32, device=dev)
    bt = table_tensor(g4.decode_blocks).to(dev)
    o = torch.empty_like(q)
    for name, window in (("decode_attn_config4_global", -1), ("decode_attn_config4_window512", 512)):
        ws = ops.decode_workspace(b, hq, d, dev)
        ops.decode_plan(lens, window, hq, hkv, d, ws, block_table=bt, block_size=256)
        ms = graph_time_ms(lambda: [ops.decode_attn(q, gp[0], gp[1], lens, bt, d ** -0.5, window, ws, out=o) for gp in gpools],
                           len(gpools))
        byts = decode_kv_bytes(GEMMA3_1B, g4.decode_ctx, window)
        gbs = byts / ms / 1e6
        out[name] = {"GB/s": round(gbs, 1), "us": round(ms * 1e3, 1), "bytes": byts,
                     "frac_of_measured_hbm": round(gbs / peaks["hbm_gbs"], 4)}
    return out


def sampler_legs(dev, peaks):
    """The sampler over Qwen3's vocabulary: the 512-row and the 64-row decode batch, greedy and top-k/top-p."""
    from mini_vllm_b200 import ops
    out = {}
    vocab = 151936
    for rows in (512, 64):
        bufs = [torch.randn(rows, vocab, device=dev).to(torch.bfloat16) for _ in range(max(2, min(16, int(600e6 / (rows * vocab * 2)))))]
        temps = torch.full((rows,), 0.8, device=dev)
        topk = torch.full((rows,), 50, dtype=torch.int32, device=dev)
        topp = torch.full((rows,), 0.9, device=dev)
        for name, call in ((f"sample_greedy_{rows}", lambda x: ops.sample(x)),
                           (f"sample_top50_p0.9_{rows}", lambda x: ops.sample(x, temps, topk, 1, 0, top_p=topp))):
            ms = graph_time_ms(lambda: [call(x) for x in bufs], len(bufs))       # distinct buffers: nothing comes from L2
            byts = rows * vocab * 2
            out[name] = {"GB/s": round(byts / ms / 1e6, 1), "us": round(ms * 1e3, 1), "bytes": byts,
                         "frac_of_measured_hbm": round(byts / ms / 1e6 / peaks["hbm_gbs"], 4)}
    return out


def config3_engine_step(mixed: bool) -> dict:
    """Config 3 through the engine (28 layers): 240 requests decoding at contexts U[128,4096] when 16 prompts
    arrive, 8 of them sharing a resident 512-token prefix (prefix cache on).  With mixed steps that is ONE
    forward pass; the reference's scheduler makes it a prefill step followed by a decode step."""
    import dataclasses
    from mini_vllm_b200.engine.engine import Engine
    case, g = config3()
    cfg = Config(hf_config=qwen3_shape(), kv_cache_num_blocks=2400, max_num_batched_seqs=512, max_graph_batch_size=256,
                 max_num_batched_tokens=20480, enable_prefix_cache=True, enable_mixed_steps=mixed,
                 gpu_memory_utilization=0.85, use_cuda_graph=True, seed=0)
    eng = Engine(cfg)
    vocab = cfg.hf_config.vocab_size
    tok = lambda n: torch.randint(0, vocab, (int(n),), generator=g).tolist()
    long_run = SamplingParams(max_tokens=4096, ignore_eos=True)
    shared = tok(512)
    warm = eng.submit(shared + tok(8), SamplingParams(max_tokens=1, ignore_eos=True))   # leaves the prefix resident
    while not eng.finished:
        eng.step()
    for c in case.decode_ctx:                      # the decoding population: prompts one token short of the context
        eng.submit(tok(c - 1), long_run)
    while eng.scheduler.waiting:
        eng.step()
    for _ in range(3):                             # settle: a few decode steps (graphs warm)
        eng.step()
    for i, (n, c) in enumerate(zip(case.prefill_lens, case.prefill_cached)):
        eng.submit((shared if c else []) + tok(n - c), long_run)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    steps, new_tokens, kinds = 0, 0, []
    while eng.scheduler.waiting or (not mixed and kinds[-1] != 1):   # the plain scheduler needs a decode step after
        b = eng.step()
        kinds.append(b.type)
        bp = len(b.requests) - b.num_decode
        new_tokens += sum(len(r.tokens) - 1 - r.num_cached_tokens for r in b.requests[:bp]) + b.num_decode
        steps += 1
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    eng.executor.check_device_status()
    return {"mixed_steps": mixed, "steps": steps, "step_types": kinds, "ms": round(ms, 3), "tokens": new_tokens,
            "tokens_per_s": round(new_tokens / ms * 1e3, 1)}


def config4_engine_step() -> dict:
    """Config 4 through the engine: Gemma3-1B shapes (26 layers, 4 global / 22 window-512), 128 requests
    decoding at contexts U[512,4096].  Device time of a decode step = (job with 65 generated tokens - job with
    1) / 64, both through the pipelined loop with CUDA graphs."""
    from mini_vllm_b200.config import gemma3_shape
    from mini_vllm_b200.engine.engine import Engine
    case, g = config4()
    cfg = Config(hf_config=gemma3_shape(), kv_cache_num_blocks=1400, max_num_batched_seqs=128, max_graph_batch_size=128,
                 max_num_batched_tokens=16384, gpu_memory_utilization=0.85, use_cuda_graph=True, seed=0)
    eng = Engine(cfg)
    vocab = cfg.hf_config.vocab_size
    prompts = [torch.randint(0, vocab, (int(c) - 1,), generator=g).tolist() for c in case.decode_ctx]
    times = {}
    for n in (1, 65, 1, 65):
        eng.generate(prompts, SamplingParams(max_tokens=n, ignore_eos=True), use_tqdm=False)
        times[n] = eng.last_job_device_ms
    step_ms = (times[65] - times[1]) / 64
    ctx_mid = [c + 32 for c in case.decode_ctx]
    byts = 4 * decode_kv_bytes(GEMMA3_1B, ctx_mid, -1) + 22 * decode_kv_bytes(GEMMA3_1B, ctx_mid, 512)
    return {"decode_step_ms": round(step_ms, 4), "sequences": len(prompts), "kv_bytes_per_step": byts,
            "kv_GB/s_over_whole_step": round(byts / step_ms / 1e6, 1), "tokens_per_s": round(len(prompts) / step_ms * 1e3, 1),
            "prefill_job_ms": round(times[1], 2)}


def config2_parity() -> dict:
    """First-32-token greedy identity on the real config-2 shape against the committed reference tokens
    (tests/golden/config2_tokens.npz: the reference's own engine loop on a B200, prompts screened for a top-1/top-2
    margin of more than one bf16 step at every step of the reference)."""
    import numpy as np
    from mini_vllm_b200.engine.engine import Engine
    z = np.load(ROOT / "tests" / "golden" / "config2_tokens.npz")
    cuts = np.concatenate([[0], np.cumsum(z["prompt_lens"])])
    prompts = [z["prompts_flat"][a:b].tolist() for a, b in zip(cuts[:-1], cuts[1:])]
    eng = Engine(build_config("config2"))
    out = eng.generate(prompts, SamplingParams(max_tokens=32, ignore_eos=True), use_tqdm=False)
    got = np.asarray([o["tokens"] for o in out], dtype=np.int32)
    same = (got == z["ref_tokens"]).all(axis=1)
    return {"prompts": len(prompts), "tokens_per_prompt": 32, "identical_prompts": int(same.sum()),
            "identical_tokens": int((got == z["ref_tokens"]).sum()), "reference": str(z["reference_kind"]),
            "min_reference_margin_bf16_steps": float(z["ref_margin_ulps"].min()),
            "screen": {"candidates": int(z["candidates"]), "pass_product_margin": int(z["pass_product_margin"]),
                       "pass_both_margins": int(z["pass_both_margins"]),
                       "differ_after_screen": int(z["mismatches_after_screen"])},
            "unscreened_identical_of_64": int(z["unscreened_identical"])}


# ---- CPU leg: the oracle restatement of the reference path on the host cores ------------------------
class CpuReference:
    """The oracle model (restatement of the reference's PyTorch path, pinned to the reference's own engine loop by
    tests/test_reference_engine.py) on the host cores.  Built once; ``sample()`` runs one bounded sample of the
    workload: the first requests of the share until ``prompt_tokens`` prompt tokens are reached (at least two
    requests), full prompts, ``n_dec`` generated tokens each, through the scheduler like any job."""

    def __init__(self, workload: str, prompt_tokens: int = 1200, n_dec: int = 16, seed: int = 0):
        from mini_vllm_b200.models.loader import load_model
        from oracle.model import OracleExecutor, OracleModel, reference_names
        self.threads = os.cpu_count() or 1
        torch.set_num_threads(self.threads)
        hf = qwen3_shape()
        self.cfg = Config(hf_config=hf, kv_cache_num_blocks=160, max_num_batched_seqs=8, use_cuda_graph=False, seed=seed)
        model = load_model(self.cfg, device="cpu")
        weights = reference_names(dict(model.state_dict()), "qwen3", hf)
        del model
        self.executor = OracleExecutor(OracleModel(weights, hf, "qwen3", 160, 256, device="cpu"), 256)
        reqs, total = [], 0
        for r in workload_requests(workload):
            if len(reqs) >= 2 and total >= prompt_tokens:
                break
            if len(r.prompt) > 2048:                 # keep one sample to seconds: the longest prompts are skipped
                continue
            reqs.append(r)
            total += len(r.prompt)
        self.reqs, self.n_dec = reqs, n_dec
        self.describe = (f"{len(reqs)} requests of the workload ({total} prompt tokens, prompts over 2048 skipped), "
                         f"{n_dec} generated tokens each, bf16 weights, prefill+decode tokens / wall time "
                         "(per-token extrapolation; prefill-heavy, which favours the CPU)")

    def sample(self) -> tuple[int, float]:
        from mini_vllm_b200.engine.request import Request
        from mini_vllm_b200.scheduler.scheduler import Scheduler
        sch = Scheduler(self.cfg)
        for r in self.reqs:
            sch.submit(Request(r.prompt, SamplingParams(max_tokens=self.n_dec, ignore_eos=True)))
        t0 = time.perf_counter()
        tokens = 0
        while not sch.finished:
            batch = sch.schedule()
            out = self.executor.execute(batch)
            tokens += sum(len(r.tokens) - r.num_cached_tokens for r in batch.requests) if batch.type == 0 else len(out)
            sch.update(batch, out)
        return tokens, time.perf_counter() - t0


def workload_config(workload: str, world: int, requests_per_gpu: int, tokens_per_step: int, mixed: bool = False) -> dict:
    """The ``config`` object of the bench line: both arms print the same keys and values for the same run."""
    return {"workload": WORKLOADS[workload] + (", mixed steps" if mixed else ""), "requests_per_gpu": requests_per_gpu,
            "parallelism": f"replicas x{world}",
            "l2": "KV pool (28 layers, >126 MB per step) exceeds L2; kernel legs rotate distinct pools",
            "tokens_per_step_all_gpus": tokens_per_step}


def reference_arm(args):
    """The reference's path on the host cores (rank 0 only): ``--warmup`` untimed and exactly ``--steps`` timed
    bounded samples; ``ms_per_step`` x ``steps`` is the time really spent in the timed region."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    cpu = CpuReference(args.workload)
    for _ in range(args.warmup):
        cpu.sample()
    tokens, secs = 0, 0.0
    for _ in range(args.steps):
        n, dt = cpu.sample()
        tokens += n
        secs += dt
    value = tokens / secs
    mine = workload_requests(args.workload, world, 0)
    per_step_all = sum(len(r.prompt) + r.max_tokens for k in range(world) for r in workload_requests(args.workload, world, k))
    config = workload_config(args.workload, world, len(mine), per_step_all)
    config["sample"] = cpu.describe
    line = {"impl": "reference", "metric": METRIC, "value": round(value, 2), "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(1e3 * secs / args.steps, 1),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config,
            "cpu_baseline": {"value": round(value, 2), "unit": "tokens/s", "cores": cpu.threads, "kind": "port",
                             "sample": cpu.describe, "tokens_per_sample": tokens // args.steps},
            "e2e": {"value": round(value, 2), "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-strong-scaling", action="store_true",
                    help="skip the extra N=1 job over all 4096 config-5 requests (about a minute)")
    ap.add_argument("--workload", default="config5", choices=["config5", "config2"],
                    help="config5 (default): 512 requests per GPU, prompts log-uniform [32,4096], outputs "
                         "U[64,1024]; config2: 64 requests per GPU, prompt U[100,1024], total <= 1024")
    ap.add_argument("--kernel-legs", nargs="?", const="all", default=None, metavar="LEGS",
                    help="only the fixed single-kernel cases (one 2.3 GB pool), then exit; optionally a comma list out "
                         "of " + ",".join(LEGS) + " to keep a profiler capture small")
    ap.add_argument("--no-fused-head", action="store_true",
                    help="variant: lm_head and the sampler as two kernels on every step (Config.fused_greedy_head=False)")
    ap.add_argument("--mixed-steps", action="store_true",
                    help="variant: prompts join steps of running decodes (Config.enable_mixed_steps)")
    ap.add_argument("--config3-step", action="store_true",
                    help="engine-level config 3: 16 prefix-cached prompts arriving among 240 decodes, as one mixed "
                         "step and as the reference's two steps")
    ap.add_argument("--config2-parity", action="store_true",
                    help="first-32-token greedy identity with the reference engine's committed tokens on the 28-layer "
                         "config-2 model (64 screened prompts)")
    ap.add_argument("--config4-step", action="store_true",
                    help="engine-level config 4: a decode step of 128 sequences on Gemma3-1B shapes")
    ap.add_argument("--engine-steps", type=int, default=0,
                    help="profiling aid: prefill + N decode steps of the workload without CUDA graphs, then exit")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.config3_step:
        torch.cuda.set_device(0)
        out = []
        for mixed in (True, False):
            out.append(config3_engine_step(mixed))
            torch.cuda.empty_cache()
        print(json.dumps({"config3_engine_step": out}))
        return
    if args.config2_parity:
        torch.cuda.set_device(0)
        print(json.dumps({"config2_parity": config2_parity()}))
        return
    if args.config4_step:
        torch.cuda.set_device(0)
        print(json.dumps({"config4_engine_step": config4_engine_step()}))
        return
    if args.kernel_legs:
        peaks, _ = measured_peaks()
        legs = LEGS if args.kernel_legs == "all" else tuple(args.kernel_legs.split(","))
        unknown = [x for x in legs if x not in LEGS]
        if unknown:
            ap.error(f"unknown kernel legs {unknown}; choose from {LEGS}")
        print(json.dumps(kernel_extras(torch.device("cuda", 0), peaks, nl=1, legs=legs)))
        return
    if args.engine_steps:
        import dataclasses
        from mini_vllm_b200.engine.engine import Engine
        torch.cuda.set_device(0)
        eng = Engine(dataclasses.replace(build_config(args.workload), use_cuda_graph=False))   # every kernel its own launch
        for r in workload_requests(args.workload):
            eng.submit(r.prompt, SamplingParams(max_tokens=r.max_tokens, ignore_eos=True))
        done = 0
        while done < args.engine_steps:
            done += eng.step().type == 1
        torch.cuda.synchronize()
        print(json.dumps({"prefill_steps": eng.metrics.prefill_steps, "decode_steps": eng.metrics.decode_steps}))
        return

    from mini_vllm_b200 import ops
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    peaks, peak_kind = measured_peaks()

    mine = workload_requests(args.workload, world, rank)
    engine = build_engine(local_rank, args.workload, mixed_steps=args.mixed_steps, fused_head=not args.no_fused_head)
    dev = engine.executor.device
    # At N > 1 the job goes through the host dispatcher: rank 0 holds every request of the job (the shares of all
    # ranks), scatters them by token cost over a gloo group, and gets the completions back.
    group, job = None, mine
    if dist is not None:
        group = dist.new_group(backend="gloo")
        job = None
        if rank == 0:
            job = [r for k in range(world) for r in workload_requests(args.workload, world, k)]

    def sync_all():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(args.warmup):
        run_job(engine, job, group=group)
    sampler = ClockSampler(local_rank)
    contexts = []
    ex = engine.executor
    sync_all()
    if rank == 0:
        sampler.start()
    launches0, h2d0, d2h0 = ops.LaunchCounter.total, ex.h2d_bytes, ex.d2h_bytes
    steps0 = engine.metrics.prefill_steps + engine.metrics.decode_steps
    t0 = time.perf_counter()
    tok = 0
    cuda_ms = 0.0
    for i in range(args.steps):
        n, wall, ms = run_job(engine, job, contexts if (rank == 0 and i == args.steps - 1) else None, group=group)
        tok += n
        cuda_ms += ms
    sync_all()
    wall_total = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else None
    launches = ops.LaunchCounter.total - launches0
    engine_steps = engine.metrics.prefill_steps + engine.metrics.decode_steps - steps0
    h2d, d2h = ex.h2d_bytes - h2d0, ex.d2h_bytes - d2h0

    stats = torch.tensor([cuda_ms, wall_total * 1e3, float(tok), float(launches)], dtype=torch.float64, device=dev)
    if dist is not None:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        cuda_ms_max, wall_ms_max, tok_all, launches_all = mx[0].item(), mx[1].item(), sm[2].item(), sm[3].item()
    else:
        cuda_ms_max, wall_ms_max, tok_all, launches_all = cuda_ms, wall_total * 1e3, float(tok), float(launches)

    # Strong-scaling reference point, N = 1 only: the whole 4096-request job of config 5 on this one GPU, once.
    strong = None
    if world == 1 and args.workload == "config5" and not args.no_strong_scaling:
        from mini_vllm_b200.workloads import config5_requests
        n, wall, ms = run_job(engine, config5_requests(seed=0, n=4096))
        strong = {"requests": 4096, "tokens": n, "device_ms": round(ms, 1), "tokens_per_s": round(n / ms * 1e3, 1),
                  "e2e_tokens_per_s": round(n / wall, 1),
                  "note": "all of config 5 on one GPU, one job; the 8-GPU run of the same 4096 requests is the N=8 line"}

    if rank == 0:
        roof = decode_roofline(engine, contexts, peaks)
        roof["peak_kind"] = f"of {peak_kind}"
        extras = kernel_extras(dev, peaks)
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            ref = CpuReference(args.workload)
            ref.sample()                                                # warm-up (allocator, thread pool)
            n1, dt1 = ref.sample()
            n2, dt2 = ref.sample()
            cpu = {"value": round((n1 + n2) / (dt1 + dt2), 2), "unit": "tokens/s", "cores": ref.threads, "kind": "port",
                   "sample": ref.describe, "seconds": round(dt1 + dt2, 1)}
        line = {
            "metric": METRIC, "value": round(tok_all / (cuda_ms_max * 1e-3), 1), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(cuda_ms_max / args.steps, 2), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(args.workload, world, len(mine), int(tok_all / args.steps), args.mixed_steps),
            "e2e": {"value": round(tok_all / (wall_ms_max * 1e-3), 1), "unit": "tokens/s",
                    "h2d_bytes_per_step": int(h2d / max(engine_steps, 1)),
                    "d2h_bytes_per_step": int(d2h / max(engine_steps, 1)),
                    "engine_steps_per_job": engine_steps // args.steps},
            "gpu_launches": int(launches_all),
            "clocks": clocks, "roofline": roof, "kernels": extras, "cpu_baseline": cpu,
        }
        if strong is not None:
            line["strong_scaling_n1_tok_s"] = strong["tokens_per_s"]
            line["strong_scaling_n1"] = strong
        if world > 1:
            line["e2e"]["path"] = ("rank 0 holds all requests: host dispatcher scatter (gloo) -> Engine.generate on every "
                                   "rank -> gather and merge on rank 0; wall clock on rank 0")
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
