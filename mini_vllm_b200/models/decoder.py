"""Decoder-only transformer around the fused attention path (Qwen3 and Gemma3 text models).

Only the attention call-site belongs to the accelerated path; projections, norms, MLP and
embedding stay PyTorch/cuBLAS, wired the way the reference wires them:

* Qwen3 (``minivllm/models/models/qwen3.py``): pre-norm residual blocks, per-head RMSNorm on q and
  k before RoPE (``:89-92``), SwiGLU MLP, optional tied lm_head, last-token gather at prefill
  (``:215-217``).
* Gemma3 (``minivllm/models/models/gemma3.py``): ``(1 + w)`` RMSNorm computed in fp32
  (``:12-24``), sandwich norms around attention and MLP (``:152-170``), GeGLU-tanh MLP, embedding
  scaled by ``sqrt(hidden)`` (``:175-184``), a global and a local RoPE table and a sliding
  window on every layer whose index ``i`` has ``(i + 1) % 6 != 0`` (``:196-211``).

q/k/v come out of ONE packed projection (row stride != heads * head_dim) and go straight into
``FlashAttention.forward_fused_norm``: per-head RMSNorm, RoPE and the KV-cache write are one kernel that
works in place on the projection output.
"""
from __future__ import annotations

from typing import Iterable

import torch
import torch.nn.functional as F
from torch import nn

from .. import ops
from ..executor.context import Context
from .layers.attention import FlashAttention
from .layers.rotary import RotaryEmbedding


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float, unit_offset: bool):
        super().__init__()
        self.eps, self.unit_offset = eps, unit_offset
        self.weight = nn.Parameter(torch.zeros(dim) if unit_offset else torch.ones(dim))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not self.unit_offset:
            return F.rms_norm(x, (x.shape[-1],), self.weight, self.eps)
        xf = x.float()
        xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
        return (xf * (1.0 + self.weight.float())).type_as(x)


class Attention(nn.Module):
    def __init__(self, cfg, rotary: RotaryEmbedding, gemma: bool, sliding_window):
        super().__init__()
        self.hq, self.hkv, self.d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        self.q_dim, self.kv_dim = self.hq * self.d, self.hkv * self.d
        self.rotary = rotary
        scaling = (cfg.query_pre_attn_scalar if gemma else self.d) ** -0.5
        self.qkv_proj = nn.Linear(cfg.hidden_size, self.q_dim + 2 * self.kv_dim, bias=cfg.attention_bias)
        self.o_proj = nn.Linear(self.q_dim, cfg.hidden_size, bias=cfg.attention_bias)
        self.q_norm = RMSNorm(self.d, cfg.rms_norm_eps, gemma)
        self.k_norm = RMSNorm(self.d, cfg.rms_norm_eps, gemma)
        self.attn = FlashAttention(self.hq, self.d, scaling, self.hkv, sliding_window)
        self.fuse_qk_norm = True                                 # Config.fuse_qk_norm, set by the loader

    def forward(self, ctx: Context, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        q, k, v = self.qkv_proj(x).split([self.q_dim, self.kv_dim, self.kv_dim], dim=-1)
        q, k, v = q.view(-1, self.hq, self.d), k.view(-1, self.hkv, self.d), v.view(-1, self.hkv, self.d)
        if not self.fuse_qk_norm:
            # the reference's sequence (qwen3.py:89-94): stand-alone per-head norms, then RoPE + cache write in
            # the kernel whose cache contents are bit-identical to the eager rotation and copy
            o = self.attn.forward_fused(ctx, self.q_norm(q), self.k_norm(k), v, positions, self.rotary.cos_sin_cache)
            return self.o_proj(o.reshape(-1, self.q_dim))
        # per-head norms, RoPE and the KV write run as one kernel on the packed projection output
        o = self.attn.forward_fused_norm(ctx, q, k, v, positions, self.rotary.cos_sin_cache, self.q_norm.weight,
                                         self.k_norm.weight, self.q_norm.eps, self.q_norm.unit_offset)
        return self.o_proj(o.reshape(-1, self.q_dim))


class GatedMLP(nn.Module):
    def __init__(self, cfg, gemma: bool):
        super().__init__()
        self.inter, self.gemma = cfg.intermediate_size, gemma
        self.gate_up_proj = nn.Linear(cfg.hidden_size, 2 * self.inter, bias=False)
        self.down_proj = nn.Linear(self.inter, cfg.hidden_size, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.down_proj(ops.act_mul(self.gate_up_proj(x), self.inter, self.gemma))


class DecoderLayer(nn.Module):
    def __init__(self, cfg, rotary: RotaryEmbedding, gemma: bool, sliding_window):
        super().__init__()
        norm = lambda: RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, gemma)
        self.gemma = gemma
        self.self_attn = Attention(cfg, rotary, gemma, sliding_window)
        self.mlp = GatedMLP(cfg, gemma)
        self.input_layernorm, self.post_attention_layernorm = norm(), norm()
        if gemma:
            self.pre_feedforward_layernorm, self.post_feedforward_layernorm = norm(), norm()

    def forward(self, ctx: Context, x: torch.Tensor, h: torch.Tensor, positions: torch.Tensor,
                next_norm: RMSNorm, last_tokens: torch.Tensor | None = None) -> torch.Tensor:
        """``x`` is the residual stream (updated in place), ``h`` its already normalised copy for this
        layer; returns the normalised input of the next layer (``next_norm`` applied to the new ``x``).
        Each residual add is fused with the norm that follows it (and, for Gemma, with the norm on the
        branch output), which is the reference's dataflow (qwen3.py:146-155, gemma3.py:157-170).

        ``last_tokens`` (the batch's ``cu_seqlens_q``, last layer of a prefill only): the closing add and the
        final norm are computed for the last token of every sequence alone - the rows the lm_head reads
        (qwen3.py:215-217) - gathered inside the kernel; the result has one row per sequence."""
        a = self.self_attn(ctx, h, positions)
        post_mlp = None if not self.gemma else self.post_feedforward_layernorm.weight
        if not self.gemma:
            n = self.post_attention_layernorm
            h = ops.add_rmsnorm(x, a, n.weight, n.eps, False)
        else:
            n = self.pre_feedforward_layernorm
            h = ops.add_rmsnorm(x, a, n.weight, n.eps, True, y_weight=self.post_attention_layernorm.weight)
        if last_tokens is not None:
            return ops.add_rmsnorm_last_tokens(x, self.mlp(h), next_norm.weight, next_norm.eps, self.gemma, last_tokens,
                                               y_weight=post_mlp)
        return ops.add_rmsnorm(x, self.mlp(h), next_norm.weight, next_norm.eps, self.gemma, y_weight=post_mlp)


class DecoderLM(nn.Module):
    """``forward(ctx, input_ids, positions) -> logits`` (one row per sequence at prefill)."""

    family = "qwen3"

    def __init__(self, cfg):
        super().__init__()
        gemma = self.family == "gemma3"
        self.config, self.gemma = cfg, gemma
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        if gemma:   # applied in the weight dtype, like gemma3.py:175-184
            self.register_buffer("embed_scale", torch.tensor(float(cfg.hidden_size) ** 0.5), persistent=False)
        else:
            self.embed_scale = None
        self.rotary = RotaryEmbedding(cfg.head_dim, cfg.max_position_embeddings, cfg.rope_theta)
        self.rotary_local = (RotaryEmbedding(cfg.head_dim, cfg.max_position_embeddings, cfg.rope_local_base_freq)
                             if gemma else None)
        # The reference hands its attention layer (sliding_window, -1) and that layer's contract reads the
        # first number as "tokens to the left of the query" (gemma3.py:66-69, attention.py:56-60): a query
        # then sees sliding_window + 1 keys.  Hugging Face counts the query itself in the window
        # (sliding_window keys); configs read from a checkpoint ask for that with sliding_window_counts_query.
        left = (cfg.sliding_window - (1 if getattr(cfg, "sliding_window_counts_query", False) else 0)) if gemma else -1
        layers = []
        for i in range(cfg.num_hidden_layers):
            local = gemma and (i + 1) % 6 != 0
            layers.append(DecoderLayer(cfg, self.rotary_local if local else self.rotary, gemma,
                                       (left, -1) if local else (-1, -1)))
        self.layers = nn.ModuleList(layers)
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, gemma)
        self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False)
        if cfg.tie_word_embeddings:
            self.lm_head.weight = self.embed_tokens.weight

    def forward(self, ctx: Context, input_ids: torch.Tensor, positions: torch.Tensor, head: bool = True) -> torch.Tensor:
        """Logits, one row per sequence (``head=True``, the reference's contract), or the rows the lm_head would
        read - final norm applied, last token of every sequence at prefill - for a caller that runs the head
        itself (``greedy_tokens`` or ``lm_head``)."""
        x = self.embed_tokens(input_ids)
        if self.embed_scale is not None:
            x = x * self.embed_scale.to(x.dtype)
        x = x.contiguous()
        h = self.layers[0].input_layernorm(x)
        last = len(self.layers) - 1
        for i, layer in enumerate(self.layers):
            nxt = self.layers[i + 1].input_layernorm if i < last else self.norm
            # at prefill the lm_head reads one row per sequence: the last layer's closing add + final norm gather
            # those rows themselves instead of normalising every token and indexing afterwards
            h = layer(ctx, x, h, positions, nxt, ctx.cu_seqlens_q if (i == last and ctx.prefill) else None)
        return self.lm_head(h) if head else h                  # the final norm is already applied

    def greedy_tokens(self, hidden_rows: torch.Tensor, scratch: torch.Tensor, out: torch.Tensor | None = None,
                      scatter_table: torch.Tensor | None = None, scatter_index: torch.Tensor | None = None,
                      status: torch.Tensor | None = None) -> torch.Tensor:
        """``argmax(lm_head(hidden_rows))`` in one kernel: the logits are never written (qwen3.py:215-219 followed
        by sampler.py:31 for requests without top-k / top-p)."""
        return ops.lm_head_argmax(hidden_rows, self.lm_head.weight, scratch, out=out, scatter_table=scatter_table,
                                  scatter_index=scatter_index, status=status)

    # ---- weights ---------------------------------------------------------------------------------
    @torch.no_grad()
    def init_random(self, seed: int, std: float = 0.02) -> None:
        """N(0, std) for every Linear/Embedding weight from a CPU generator; norm gains keep their defaults."""
        g = torch.Generator(device="cpu").manual_seed(seed)
        seen = set()
        for name, p in self.named_parameters():
            if "norm" in name or id(p) in seen:
                continue
            seen.add(id(p))
            p.copy_((torch.randn(p.shape, generator=g, dtype=torch.float32) * std).to(p.dtype))

    @torch.no_grad()
    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> None:
        """Accepts Hugging Face names (separate q/k/v and gate/up) as well as packed ``qkv_proj``."""
        params = dict(self.named_parameters())
        q_dim = self.config.num_attention_heads * self.config.head_dim
        kv_dim = self.config.num_key_value_heads * self.config.head_dim
        inter = self.config.intermediate_size
        shard = {"q_proj": ("qkv_proj", 0, q_dim), "k_proj": ("qkv_proj", q_dim, kv_dim),
                 "v_proj": ("qkv_proj", q_dim + kv_dim, kv_dim),
                 "gate_proj": ("gate_up_proj", 0, inter), "up_proj": ("gate_up_proj", inter, inter)}
        for name, w in weights:
            name = name.removeprefix("model.") if name.startswith("model.") else name
            if name == "lm_head.weight" and self.config.tie_word_embeddings:
                continue
            for part, (packed, start, size) in shard.items():
                if f".{part}." in name:
                    params[name.replace(part, packed)].narrow(0, start, size).copy_(w)
                    break
            else:
                if name not in params:
                    raise KeyError(f"unrecognised parameter {name}")
                params[name].copy_(w)
