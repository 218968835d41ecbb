"""Qwen3 / Gemma3 decoder forward restated functionally (PyTorch eager, any device).  TEST INFRASTRUCTURE.

Weights come as a dict with the reference modules' own parameter names (``state_dict()`` of
``Qwen3ForCausalLM`` / ``Gemma3ForCausalLM``).  Every step follows the reference line it cites;
attention and the KV write go through the oracle's gather-and-SDPA (``oracle/attention.py``,
``oracle/rope_kv.py``) exactly where the reference calls its Triton / flash-attention kernels.
Pinned against logits produced by the reference's own module code (tests/golden/*_tiny.npz).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import attention as oattn
from . import rope_kv


def _rms(x, w, eps):                       # nn.RMSNorm as used in qwen3.py:64-65,134-138,176
    return F.rms_norm(x, (x.shape[-1],), w, eps)


def _gemma_rms(x, w, eps):                 # gemma3.py:12-24
    xf = x.float()
    xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (xf * (1.0 + w.float())).type_as(x)


class OracleModel:
    def __init__(self, weights: dict, cfg, family: str, num_blocks: int, block_size: int, device="cpu",
                 use_window: bool = True):
        self.w = {k: v.to(device) for k, v in weights.items()}
        self.cfg, self.family, self.device = cfg, family, device
        self.gemma = family == "gemma3"
        self.use_window = use_window       # the reference never forwards its window (attention.py:84-91)
        d = cfg.head_dim
        self.table = rope_kv.cos_sin_table(d, cfg.max_position_embeddings, cfg.rope_theta).to(device)
        self.table_local = (rope_kv.cos_sin_table(d, cfg.max_position_embeddings, cfg.rope_local_base_freq).to(device)
                            if self.gemma else None)
        shape = (num_blocks, block_size, cfg.num_key_value_heads, d)
        self.k_cache = [torch.zeros(shape, dtype=torch.bfloat16, device=device) for _ in range(cfg.num_hidden_layers)]
        self.v_cache = [torch.zeros(shape, dtype=torch.bfloat16, device=device) for _ in range(cfg.num_hidden_layers)]

    def _attention(self, i, ctx, x, positions):
        cfg, w, p = self.cfg, self.w, f"model.layers.{i}.self_attn."
        hq, hkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        if self.gemma:                                                  # gemma3.py:88-98
            q, k, v = (F.linear(x, w[p + n + "_proj.weight"]) for n in "qkv")
            norm = _gemma_rms
        else:                                                           # qwen3.py:81-90
            q, k, v = F.linear(x, w[p + "qkv_proj.weight"]).split([hq * d, hkv * d, hkv * d], dim=-1)
            norm = _rms
        q, k, v = q.view(-1, hq, d), k.view(-1, hkv, d), v.view(-1, hkv, d)
        q, k = norm(q, w[p + "q_norm.weight"], cfg.rms_norm_eps), norm(k, w[p + "k_norm.weight"], cfg.rms_norm_eps)
        local = self.gemma and (i + 1) % 6 != 0                         # gemma3.py:210-211
        q, k = rope_kv.apply_rope(positions, q, k, self.table_local if local else self.table)
        # (sliding_window, -1) at gemma3.py:66-69 = that many keys to the left of the query; a config that
        # sets sliding_window_counts_query asks for the Hugging Face convention (the query is one of them)
        window = -1
        if local and self.use_window:
            window = cfg.sliding_window - (1 if getattr(cfg, "sliding_window_counts_query", False) else 0)
        scale = (cfg.query_pre_attn_scalar if self.gemma else d) ** -0.5
        kc, vc = self.k_cache[i], self.v_cache[i]
        if ctx["slot_mapping"] is not None and ctx["slot_mapping"].numel() == k.shape[0]:
            rope_kv.store_kvcache(k, v, kc, vc, ctx["slot_mapping"])    # attention.py:75-76
        if ctx["prefill"]:                                              # attention.py:78-87
            if ctx["block_table"] is not None:
                o = oattn.prefill(q, kc, vc, ctx["cu_seqlens_q"], ctx["cu_seqlens_k"], ctx["block_table"], scale, window)
            else:
                o = oattn.prefill(q, k, v, ctx["cu_seqlens_q"], ctx["cu_seqlens_k"], None, scale, window)
        else:                                                           # attention.py:88-91
            o = oattn.decode(q, kc, vc, ctx["cache_seqlens"], ctx["block_table"], scale, window)
        return F.linear(o.reshape(-1, hq * d), w[p + "o_proj.weight"])

    def _mlp(self, i, x):
        w, p = self.w, f"model.layers.{i}.mlp."
        gate, up = F.linear(x, w[p + "gate_proj.weight"]), F.linear(x, w[p + "up_proj.weight"])
        act = F.gelu(gate, approximate="tanh") if self.gemma else F.silu(gate)     # gemma3.py:122 / qwen3.py:119
        return F.linear(act * up, w[p + "down_proj.weight"])

    @torch.inference_mode()
    def forward(self, ctx: dict, input_ids: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        cfg, w, eps = self.cfg, self.w, self.cfg.rms_norm_eps
        x = F.embedding(input_ids, w["model.embed_tokens.weight"])
        if self.gemma:                                                  # gemma3.py:183-184
            x = x * torch.tensor(cfg.hidden_size ** 0.5).to(x.dtype).to(x.device)
        for i in range(cfg.num_hidden_layers):
            p = f"model.layers.{i}."
            if self.gemma:                                              # gemma3.py:157-170
                h = _gemma_rms(x, w[p + "input_layernorm.weight"], eps)
                h = self._attention(i, ctx, h, positions)
                x = x + _gemma_rms(h, w[p + "post_attention_layernorm.weight"], eps)
                h = self._mlp(i, _gemma_rms(x, w[p + "pre_feedforward_layernorm.weight"], eps))
                x = x + _gemma_rms(h, w[p + "post_feedforward_layernorm.weight"], eps)
            else:                                                       # qwen3.py:146-155
                x = self._attention(i, ctx, _rms(x, w[p + "input_layernorm.weight"], eps), positions) + x
                x = self._mlp(i, _rms(x, w[p + "post_attention_layernorm.weight"], eps)) + x
        x = (_gemma_rms if self.gemma else _rms)(x, w["model.norm.weight"], eps)
        if ctx["prefill"]:                                              # qwen3.py:215-217
            x = x[(ctx["cu_seqlens_q"][1:] - 1).long()].contiguous()
        head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
        return F.linear(x, head)


class OracleExecutor:
    """``execute(batch) -> list[int]`` like ``minivllm/executor/executor.py:216-225``, greedy only."""

    def __init__(self, model: OracleModel, block_size: int):
        self.model, self.block_size = model, block_size

    def execute(self, batch) -> list[int]:
        return torch.argmax(self.logits(batch), dim=-1).tolist()        # sampler.py:31

    def logits(self, batch) -> torch.Tensor:
        from . import packing
        if batch.type == 2:                                             # a mixed step is its two halves, row order kept
            from types import SimpleNamespace
            bp = len(batch.requests) - batch.num_decode
            return torch.cat([self.logits(SimpleNamespace(type=0, requests=batch.requests[:bp])),
                              self.logits(SimpleNamespace(type=1, requests=batch.requests[bp:]))])
        dev = self.model.device
        reqs = batch.requests
        toks, blks = [r.tokens for r in reqs], [r.blocks for r in reqs]
        if batch.type == 0:
            p = packing.build_prefill_input(toks, blks, [r.num_cached_tokens for r in reqs], self.block_size)
        else:
            p = packing.build_decode_input(toks, blks, self.block_size)
        t = lambda a: None if a is None else torch.from_numpy(a).to(dev)
        ctx = {"prefill": batch.type == 0, "slot_mapping": t(p["slot_mapping"]), "block_table": t(p["block_table"]),
               "cu_seqlens_q": t(p.get("cu_seqlens_q")), "cu_seqlens_k": t(p.get("cu_seqlens_k")),
               "cache_seqlens": t(p.get("cache_seqlens"))}
        return self.model.forward(ctx, t(p["input_ids"]), t(p["positions"]))


def reference_names(state: dict, family: str, cfg) -> dict:
    """Map the product model's packed parameter names back to the reference modules' names."""
    hq, hkv, d, inter = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.intermediate_size
    out = {}
    for name, w in state.items():
        name = name if name.startswith("lm_head") else "model." + name
        if name.endswith("gate_up_proj.weight"):
            g, u = w.split([inter, inter], dim=0)
            out[name.replace("gate_up_proj", "gate_proj")] = g
            out[name.replace("gate_up_proj", "up_proj")] = u
        elif name.endswith("qkv_proj.weight") and family == "gemma3":
            q, k, v = w.split([hq * d, hkv * d, hkv * d], dim=0)
            for n, t in zip("qkv", (q, k, v)):
                out[name.replace("qkv_proj", n + "_proj")] = t
        else:
            out[name] = w
    return out
