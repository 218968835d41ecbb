"""Generate the golden vectors under tests/golden/ by running the reference's own code.

Run once where the reference checkout is available:

    TORCHDYNAMO_DISABLE=1 python tests/golden/make_golden.py /path/to/mini-vllm

The reference is imported, never copied.  Its attention layer imports the absent
third-party ``mini_flash_attention``; a stub module with the two function names
is registered first so that ``minivllm.executor.executor`` imports.  The packing
functions run on CPU with ``pin_memory``/``.cuda`` turned into no-ops.
``TORCHDYNAMO_DISABLE=1`` makes ``torch.compile`` a no-op so the reference's
``RotaryEmbedding.forward`` runs its eager arithmetic.

Outputs (all small): packing.npz, rope.npz, block_manager.json, scheduler.json,
hashes.json, qwen3_tiny.npz, gemma3_tiny.npz.
"""
from __future__ import annotations

import json
import os
import sys
import types
from pathlib import Path
from types import SimpleNamespace

os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
sys.path.insert(0, str(REPO))
if len(sys.argv) < 2:
    sys.exit("usage: make_golden.py /path/to/mini-vllm   (a checkout of w4096/mini-vllm)")
REF = Path(sys.argv[1])
sys.path.insert(0, str(REF))

from oracle import attention as oattn  # noqa: E402  (the stub kernels the reference model runs around)

# ---- stub for the un-vendored attention package -------------------------------------------
stub = types.ModuleType("mini_flash_attention")
_CTX = {}


def _varlen(q, k, v, max_seqlen_q, cu_seqlens_q, max_seqlen_k, cu_seqlens_k, causal=True):
    bt = _CTX.get("block_table")
    return oattn.prefill(q, k, v, cu_seqlens_q, cu_seqlens_k, block_table=bt)


def _with_kvcache(q, k_cache, v_cache, cache_seqlens, block_table):
    return oattn.decode(q[:, 0], k_cache, v_cache, cache_seqlens, block_table).unsqueeze(1)


stub.flash_attn_varlen_func = _varlen
stub.flash_attn_with_kvcache = _with_kvcache
sys.modules["mini_flash_attention"] = stub

# flashinfer is imported by the reference sampler module; only the name is needed on CPU
if "flashinfer" not in sys.modules:
    try:
        import flashinfer.sampling  # noqa: F401
    except Exception:
        fi = types.ModuleType("flashinfer")
        fis = types.ModuleType("flashinfer.sampling")
        fis.top_k_top_p_sampling_from_logits = None
        fi.sampling = fis
        sys.modules["flashinfer"], sys.modules["flashinfer.sampling"] = fi, fis

# make Tensor.cuda and pin_memory no-ops so the packing code runs on CPU
_orig_tensor = torch.tensor
torch.tensor = lambda *a, **kw: _orig_tensor(*a, **{k: v for k, v in kw.items() if k != "pin_memory"})
torch.Tensor.cuda = lambda self, *a, **kw: self

# triton's jit decorator needs a GPU-less import path only; importing the module is enough
from minivllm.engine.request import Request  # noqa: E402
from minivllm.kvcache.block_manager import KVCacheBlockManager, KVCacheBlock  # noqa: E402
from minivllm.scheduler.scheduler import Scheduler  # noqa: E402
from minivllm.scheduler.batch import Batch  # noqa: E402
from minivllm.config.sampling import SamplingParams  # noqa: E402
from minivllm.models.layers.rotary import RotaryEmbedding  # noqa: E402
from minivllm.executor.executor import Executor  # noqa: E402

BS = 256


def rng(seed):
    return torch.Generator(device="cpu").manual_seed(seed)


def fake_self():
    return SimpleNamespace(config=SimpleNamespace(kv_cache_block_size=BS),
                           _build_block_table=Executor._build_block_table)


# ---- 1. packing ----------------------------------------------------------------------------
def packing_cases():
    out = {}
    g = rng(1)
    cases = {
        # name: (lengths, shared prefix blocks per request)
        "plain": ([244, 460, 485, 165, 332, 438, 232, 320], [0] * 8),
        "edges": ([1, 255, 256, 257, 511, 512, 513, 1024], [0] * 8),
        "prefix": ([803, 81, 942, 185, 700, 513], [0, 0, 2, 0, 2, 2]),
        "single": ([300], [0]),
    }
    for name, (lens, shared) in cases.items():
        mgr = KVCacheBlockManager(64, BS, support_prefix_cache=True)
        prefix = torch.randint(0, 1000, (1024,), generator=g).tolist()
        reqs = []
        # a resident request that owns the shared prefix blocks
        if any(shared):
            owner = Request(prefix[:max(shared) * BS] + [7])
            mgr.allocate_blocks_for_prefill(owner)
        for n, sh in zip(lens, shared):
            body = torch.randint(0, 1000, (n,), generator=g).tolist()
            toks = prefix[:sh * BS] + body[:n - sh * BS]
            r = Request(toks)
            mgr.allocate_blocks_for_prefill(r)
            reqs.append(r)
        ids, ctx = Executor._build_prefill_input(fake_self(), reqs)
        pre = f"{name}/prefill/"
        out[pre + "tok_len"] = np.asarray([len(r.tokens) for r in reqs], np.int32)
        out[pre + "cached"] = np.asarray([r.num_cached_tokens for r in reqs], np.int32)
        out[pre + "tokens_flat"] = np.asarray([t for r in reqs for t in r.tokens], np.int32)
        out[pre + "blocks_flat"] = np.asarray([b for r in reqs for b in r.blocks], np.int32)
        out[pre + "nblocks"] = np.asarray([len(r.blocks) for r in reqs], np.int32)
        out[pre + "input_ids"] = ids.numpy()
        out[pre + "positions"] = ctx.positions.numpy()
        out[pre + "slot_mapping"] = ctx.slot_mapping.numpy()
        out[pre + "cu_seqlens_q"] = ctx.cu_seqlens_q.numpy()
        out[pre + "cu_seqlens_k"] = ctx.cu_seqlens_k.numpy()
        out[pre + "max_seqlen"] = np.asarray([ctx.max_seqlen_q, ctx.max_seqlen_k], np.int32)
        if ctx.block_table is not None:
            out[pre + "block_table"] = ctx.block_table.numpy()
        # decode step right after: every request gets one more token (and maybe a block)
        for r in reqs:
            r.state = Request.RUNNING
            r.append_output_token(int(torch.randint(0, 1000, (1,), generator=g)))
            mgr.allocate_block_for_decode(r)
        ids, ctx = Executor._build_decode_input(fake_self(), reqs)
        pre = f"{name}/decode/"
        out[pre + "tok_len"] = np.asarray([len(r.tokens) for r in reqs], np.int32)
        out[pre + "last_token"] = np.asarray([r.tokens[-1] for r in reqs], np.int32)
        out[pre + "blocks_flat"] = np.asarray([b for r in reqs for b in r.blocks], np.int32)
        out[pre + "nblocks"] = np.asarray([len(r.blocks) for r in reqs], np.int32)
        out[pre + "input_ids"] = ids.numpy()
        out[pre + "positions"] = ctx.positions.numpy()
        out[pre + "slot_mapping"] = ctx.slot_mapping.numpy()
        out[pre + "cache_seqlens"] = ctx.cache_seqlens.numpy()
        out[pre + "block_table"] = ctx.block_table.numpy()
    np.savez_compressed(HERE / "packing.npz", **out)


# ---- 2. rope -------------------------------------------------------------------------------
def rope_cases():
    out = {}
    g = rng(2)
    for name, (hq, hkv, d, theta, max_pos) in {
        "qwen3": (16, 8, 128, 1e6, 4096),
        "gemma3_global": (4, 1, 256, 1e6, 8192),
        "gemma3_local": (4, 1, 256, 1e4, 8192),
    }.items():
        rot = RotaryEmbedding(d, max_pos, theta)
        t = 53
        pos = torch.randint(0, max_pos, (t,), generator=g)
        pos[0], pos[1] = 0, max_pos - 1
        q = torch.randn(t, hq, d, generator=g).to(torch.bfloat16)
        k = torch.randn(t, hkv, d, generator=g).to(torch.bfloat16)
        q2, k2 = rot(pos, q, k)
        out[name + "/meta"] = np.asarray([hq, hkv, d, max_pos], np.int64)
        out[name + "/theta"] = np.asarray([theta], np.float64)
        out[name + "/positions"] = pos.numpy()
        out[name + "/table_rows"] = rot.cos_sin_cache[pos].numpy()
        for nm, x in (("q", q), ("k", k), ("q_out", q2), ("k_out", k2)):
            out[f"{name}/{nm}"] = x.view(torch.int16).numpy()
    np.savez_compressed(HERE / "rope.npz", **out)


# ---- 3. block manager + hashes -------------------------------------------------------------
def block_manager_trace():
    g = rng(3)
    events = []
    mgr = KVCacheBlockManager(48, BS, support_prefix_cache=True)
    base = torch.randint(0, 50000, (2048,), generator=g).tolist()
    live = []
    script = [("alloc", 700, 0), ("alloc", 600, 2), ("alloc", 1024, 4), ("free", 0), ("alloc", 900, 2),
              ("grow", 1, 300), ("free", 1), ("alloc", 513, 2), ("alloc", 512, 2), ("free", 2), ("free", 3),
              ("alloc", 1500, 4), ("alloc", 256, 1), ("free", 4), ("alloc", 768, 3)]
    for ev in script:
        if ev[0] == "alloc":
            _, n, shared = ev
            body = torch.randint(0, 50000, (n,), generator=g).tolist()
            toks = (base[:shared * BS] + body)[:n] if shared * BS < n else base[:n]
            r = Request(toks)
            ok = mgr.can_allocate_new_block(r)
            rec = {"op": "alloc", "tokens": toks, "can": bool(ok)}
            if ok:
                mgr.allocate_blocks_for_prefill(r)
                r.state = Request.RUNNING
                live.append(r)
                rec.update(blocks=list(r.blocks), cached=r.num_cached_tokens)
            events.append(rec)
        elif ev[0] == "grow":
            _, idx, steps = ev
            r = live[idx]
            new = torch.randint(0, 50000, (steps,), generator=g).tolist()
            blocks_after = []
            for t in new:
                r.append_output_token(t)
                mgr.cache_block_if_needed(r)
                if mgr.can_allocate_new_block(r):
                    mgr.allocate_block_for_decode(r)
                blocks_after.append(len(r.blocks))
            events.append({"op": "grow", "index": idx, "tokens": new, "blocks": list(r.blocks),
                           "nblocks_after_each": blocks_after})
        else:
            _, idx = ev
            r = live[idx]
            mgr.deallocate(r)
            events.append({"op": "free", "index": idx})
        events[-1]["free_ids"] = list(mgr.free_block_ids)
        events[-1]["used_ids"] = sorted(mgr.used_block_ids)
    (HERE / "block_manager.json").write_text(json.dumps({"capacity": 48, "block_size": BS, "events": events}))

    hashes = {
        "kat": [
            {"tokens": [1, 2, 3], "prefix": -1, "hash": KVCacheBlock.compute_hash([1, 2, 3])},
            {"tokens": [1, 2, 3], "prefix": 7, "hash": KVCacheBlock.compute_hash([1, 2, 3], 7)},
            {"tokens": base[:256], "prefix": -1, "hash": KVCacheBlock.compute_hash(base[:256])},
            {"tokens": base[256:512], "prefix": KVCacheBlock.compute_hash(base[:256]),
             "hash": KVCacheBlock.compute_hash(base[256:512], KVCacheBlock.compute_hash(base[:256]))},
        ],
        "fresh_pool_first_ids": None,
    }
    m2 = KVCacheBlockManager(10240, BS)
    r = Request(list(range(600)))
    m2.allocate_blocks_for_prefill(r)
    hashes["fresh_pool_first_ids"] = list(r.blocks)
    (HERE / "hashes.json").write_text(json.dumps(hashes))


# ---- 4. scheduler trace --------------------------------------------------------------------
def scheduler_trace():
    """Drive the reference Scheduler with a deterministic fake model (token = f(request, step))."""
    traces = {}
    for name, (cap, max_seqs, max_tokens_batch, prefix) in {
        "roomy": (64, 8, 4096, False),
        "tight_preempt": (12, 6, 2048, False),
        "prefix_cache": (40, 8, 4096, True),
    }.items():
        g = rng(4)
        cfg = SimpleNamespace(max_num_batched_seqs=max_seqs, max_num_batched_tokens=max_tokens_batch,
                              eos_token_ids={9999}, kv_cache_num_blocks=cap, kv_cache_block_size=BS)
        sch = Scheduler(cfg)
        if prefix:
            sch.block_manager.support_prefix_cache = True
        shared = torch.randint(0, 9000, (600,), generator=g).tolist()
        prompts, sps = [], []
        for i in range(14):
            n = int(torch.randint(20, 700, (1,), generator=g))
            body = torch.randint(0, 9000, (n,), generator=g).tolist()
            if prefix and i % 2 == 0:
                body = shared[:512] + body[:max(1, n - 300)]
            mt = int(torch.randint(5, 300, (1,), generator=g))
            prompts.append(body)
            sps.append({"max_tokens": mt, "ignore_eos": bool(i % 3)})
        base_id = None
        reqs = []
        for p, sp in zip(prompts, sps):
            r = Request(p, SamplingParams(max_tokens=sp["max_tokens"], ignore_eos=sp["ignore_eos"]))
            base_id = r.id if base_id is None else base_id
            reqs.append(r)
            sch.submit(r)
        steps = []
        n_step = 0
        while not sch.finished:
            batch = sch.schedule()
            assert batch is not None
            rows = [{"rid": r.id - base_id, "len": len(r.tokens), "cached": r.num_cached_tokens,
                     "blocks": list(r.blocks)} for r in batch.requests]
            # fake model: token depends on request and its length; EOS (9999) now and then
            toks = [9999 if (r.id - base_id + len(r.tokens)) % 97 == 0 else (r.id * 31 + len(r.tokens) * 7) % 9000
                    for r in batch.requests]
            sch.update(batch, toks)
            steps.append({"type": batch.type, "rows": rows, "tokens": toks,
                          "waiting": [r.id - base_id for r in sch.waiting],
                          "running": [r.id - base_id for r in sch.running]})
            n_step += 1
            assert n_step < 5000
        traces[name] = {"capacity": cap, "max_seqs": max_seqs, "max_tokens": max_tokens_batch,
                        "prefix_cache": prefix, "prompts": prompts, "sampling": sps, "steps": steps,
                        "completions": [r.completion_tokens for r in reqs]}
    (HERE / "scheduler.json").write_text(json.dumps(traces))


# ---- 5. tiny models through the reference's own module code --------------------------------
def tiny_models():
    from minivllm.executor.context import Context
    from minivllm.models.models.qwen3 import Qwen3ForCausalLM
    from minivllm.models.models.gemma3 import Gemma3ForCausalLM

    def run(model_cls, cfg, fname, seed):
        torch.manual_seed(seed)
        torch.set_default_dtype(torch.bfloat16)
        model = model_cls(cfg)
        torch.set_default_dtype(torch.float32)
        g = rng(seed)
        with torch.no_grad():
            for n, p in model.named_parameters():
                if "norm" in n:
                    continue                       # norm gains stay at the constructor defaults
                p.copy_(torch.randn(p.shape, generator=g) * 0.05)
        nblocks = 8
        caches = []
        for m in model.modules():
            if hasattr(m, "k_cache") and hasattr(m, "v_cache"):
                m.k_cache = torch.zeros(nblocks, BS, cfg.num_key_value_heads, cfg.head_dim, dtype=torch.bfloat16)
                m.v_cache = torch.zeros_like(m.k_cache)
                caches.append(m)
        # reference store_kvcache is a Triton kernel: route it to the eager restatement on CPU
        import minivllm.models.layers.attention as ref_attn
        from oracle.rope_kv import store_kvcache
        ref_attn.store_kvcache = store_kvcache
        lens = [37, 300, 5]
        blocks = [[5], [2, 7], [0]]
        reqs = []
        for n, b in zip(lens, blocks):
            r = Request(torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist())
            r.blocks = list(b)
            reqs.append(r)
        out = {"lens": np.asarray(lens), "blocks_flat": np.asarray([x for b in blocks for x in b]),
               "nblocks": np.asarray([len(b) for b in blocks]),
               "tokens_flat": np.asarray([t for r in reqs for t in r.tokens])}
        with torch.inference_mode():
            ids, ctx = Executor._build_prefill_input(fake_self(), reqs)
            _CTX["block_table"] = None
            logits = model(ctx, ids, ctx.positions)
            out["prefill_logits"] = logits.float().numpy()
            toks = torch.argmax(logits, -1).tolist()
            dec = []
            for step in range(3):
                for r, t in zip(reqs, toks):
                    r.append_output_token(t)
                ids, ctx = Executor._build_decode_input(fake_self(), reqs)
                logits = model(ctx, ids, ctx.positions)
                dec.append(logits.float().numpy())
                toks = torch.argmax(logits, -1).tolist()
            out["decode_logits"] = np.stack(dec)
        sd = {k: v.float().numpy() for k, v in model.state_dict().items()}
        np.savez_compressed(HERE / fname, **out, **{"w/" + k: v for k, v in sd.items()})

    qcfg = SimpleNamespace(architectures=["Qwen3ForCausalLM"], hidden_size=64, num_attention_heads=4,
                           num_key_value_heads=2, head_dim=32, num_hidden_layers=2, intermediate_size=128,
                           vocab_size=211, rms_norm_eps=1e-6, attention_bias=False, rope_theta=1e6,
                           max_position_embeddings=1024, tie_word_embeddings=True, dtype=torch.bfloat16)
    run(Qwen3ForCausalLM, qcfg, "qwen3_tiny.npz", 5)
    gcfg = SimpleNamespace(architectures=["Gemma3ForCausalLM"], hidden_size=64, num_attention_heads=4,
                           num_key_value_heads=1, head_dim=32, num_hidden_layers=6, intermediate_size=128,
                           vocab_size=211, rms_norm_eps=1e-6, attention_bias=False, rope_theta=1e6,
                           rope_local_base_freq=1e4, query_pre_attn_scalar=32, sliding_window=512,
                           max_position_embeddings=1024, tie_word_embeddings=True, dtype=torch.bfloat16)
    run(Gemma3ForCausalLM, gcfg, "gemma3_tiny.npz", 6)


if __name__ == "__main__":
    packing_cases()
    rope_cases()
    block_manager_trace()
    scheduler_trace()
    tiny_models()
    for f in sorted(HERE.glob("*.np*")) + sorted(HERE.glob("*.json")):
        print(f.name, f.stat().st_size)
