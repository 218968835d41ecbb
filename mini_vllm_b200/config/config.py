"""Engine configuration: the reference's ``Config`` fields (minivllm/config/config.py:6-59) plus a
path-free way to describe a model, since random-init runs have no checkpoint directory.

``hf_config`` is any object with the attributes the engine reads (``architectures``, ``dtype``,
``num_hidden_layers``, ``num_attention_heads``, ``num_key_value_heads``, ``head_dim``,
``hidden_size``, ``intermediate_size``, ``vocab_size``, ``rms_norm_eps``, ``attention_bias``,
``max_position_embeddings``, ``rope_theta``, ``tie_word_embeddings``, ``eos_token_id`` and, for
Gemma3, ``query_pre_attn_scalar``, ``sliding_window``, ``rope_local_base_freq``).  When only
``model`` (a Hugging Face directory) is given it is read with ``AutoConfig`` as the reference does.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from types import SimpleNamespace
from typing import Any, Optional, Set

import torch


@dataclass
class Config:
    model: Optional[str] = None
    hf_config: Any = None
    max_model_len: int = 4096

    # scheduler
    max_num_batched_tokens: int = 16384
    max_num_batched_seqs: int = 512
    eos_token_ids: Optional[Set[int]] = None

    # kv cache
    kv_cache_num_blocks: int = 256
    kv_cache_block_size: int = 256
    gpu_memory_utilization: float = 0.5
    enable_prefix_cache: bool = False        # the reference ships with prefix caching switched off
    enable_mixed_steps: bool = False         # extension: new prompts join a step of running decodes (scheduler.py)

    # executor
    use_cuda_graph: bool = True
    max_graph_batch_size: int = 256          # largest decode batch replayed from a CUDA graph (graph.py:11)
    seed: int = 0                            # weights of a random-init model and the sampler's stream
    # True: per-head q/k RMSNorm, RoPE and the cache write run as one kernel (results within one bf16 ulp of the
    # unfused sequence).  False: stand-alone norms, then the RoPE + write kernel whose cache contents are
    # bit-identical to the reference's eager rotation and copy.
    fuse_qk_norm: bool = True
    # True: a step whose requests all sample greedily (no top-k / top-p) runs lm_head and argmax as one kernel and
    # never materialises its logits.  False: lm_head, then the sampler, as the reference does.
    fused_greedy_head: bool = True
    fused_head_max_rows: int = 256           # beyond this many rows cuBLAS + the greedy sampler are faster (measured)

    def __post_init__(self):
        if self.hf_config is None:
            if self.model is None:
                raise ValueError("Config needs either hf_config (a shape description) or model (a directory)")
            path = os.path.expanduser(self.model)
            if not os.path.isdir(path):
                raise ValueError(f"Model path {self.model} is not a directory.")
            from transformers import AutoConfig
            self.hf_config = _flatten_hf(AutoConfig.from_pretrained(path))
        if self.eos_token_ids is None:
            eos = getattr(self.hf_config, "eos_token_id", None)
            if eos is None:
                self.eos_token_ids = set()
            elif isinstance(eos, int):
                self.eos_token_ids = {eos}
            else:
                self.eos_token_ids = set(eos)
        if self.kv_cache_block_size % 128 != 0:
            raise ValueError("kv_cache_block_size must be a multiple of 128 (the prefill KV tile)")


def _flatten_hf(cfg) -> SimpleNamespace:
    """Copy the attributes the engine reads; newer transformers keep the RoPE bases in rope_parameters."""
    names = ["architectures", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim",
             "hidden_size", "intermediate_size", "vocab_size", "rms_norm_eps", "attention_bias",
             "max_position_embeddings", "tie_word_embeddings", "eos_token_id", "query_pre_attn_scalar",
             "sliding_window", "rope_theta", "rope_local_base_freq"]
    out = SimpleNamespace(**{n: getattr(cfg, n) for n in names if hasattr(cfg, n)})
    rp = getattr(cfg, "rope_parameters", None)
    if isinstance(rp, dict):
        if "rope_theta" in rp and not hasattr(out, "rope_theta"):
            out.rope_theta = rp["rope_theta"]
        full, local = rp.get("full_attention"), rp.get("sliding_attention")
        if isinstance(full, dict) and "rope_theta" in full:
            out.rope_theta = full["rope_theta"]
        if isinstance(local, dict) and "rope_theta" in local:
            out.rope_local_base_freq = local["rope_theta"]
    out.sliding_window_counts_query = True      # checkpoints follow the Hugging Face window convention
    out.dtype = getattr(cfg, "dtype", None) or getattr(cfg, "torch_dtype", None) or torch.bfloat16
    if not hasattr(out, "head_dim"):
        out.head_dim = out.hidden_size // out.num_attention_heads
    return out


def qwen3_shape(num_hidden_layers: int = 28, hidden_size: int = 1024, intermediate_size: int = 3072,
                num_attention_heads: int = 16, num_key_value_heads: int = 8, head_dim: int = 128,
                vocab_size: int = 151936, max_position_embeddings: int = 40960, rope_theta: float = 1e6,
                tie_word_embeddings: bool = True, **extra) -> SimpleNamespace:
    """Qwen3-0.6B by default."""
    return SimpleNamespace(architectures=["Qwen3ForCausalLM"], dtype=torch.bfloat16,
                           num_hidden_layers=num_hidden_layers, hidden_size=hidden_size,
                           intermediate_size=intermediate_size, num_attention_heads=num_attention_heads,
                           num_key_value_heads=num_key_value_heads, head_dim=head_dim, vocab_size=vocab_size,
                           rms_norm_eps=1e-6, attention_bias=False, max_position_embeddings=max_position_embeddings,
                           rope_theta=rope_theta, tie_word_embeddings=tie_word_embeddings, eos_token_id=None, **extra)


def gemma3_shape(num_hidden_layers: int = 26, hidden_size: int = 1152, intermediate_size: int = 6912,
                 num_attention_heads: int = 4, num_key_value_heads: int = 1, head_dim: int = 256,
                 vocab_size: int = 262144, max_position_embeddings: int = 32768, rope_theta: float = 1e6,
                 rope_local_base_freq: float = 1e4, sliding_window: int = 512, query_pre_attn_scalar: int = 256,
                 tie_word_embeddings: bool = True, **extra) -> SimpleNamespace:
    """Gemma3-1B by default."""
    return SimpleNamespace(architectures=["Gemma3ForCausalLM"], dtype=torch.bfloat16,
                           num_hidden_layers=num_hidden_layers, hidden_size=hidden_size,
                           intermediate_size=intermediate_size, num_attention_heads=num_attention_heads,
                           num_key_value_heads=num_key_value_heads, head_dim=head_dim, vocab_size=vocab_size,
                           rms_norm_eps=1e-6, attention_bias=False, max_position_embeddings=max_position_embeddings,
                           rope_theta=rope_theta, rope_local_base_freq=rope_local_base_freq,
                           sliding_window=sliding_window, query_pre_attn_scalar=query_pre_attn_scalar,
                           tie_word_embeddings=tie_word_embeddings, eos_token_id=None, **extra)
