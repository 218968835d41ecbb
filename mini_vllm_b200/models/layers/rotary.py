"""Rotary position embedding table (the rotation itself is fused into the KV-write kernel).

The table is built exactly as ``minivllm/models/layers/rotary.py:32-47`` builds it — fp32,
``[max_position_embeddings, rotary_dim] = cat(cos, sin)`` — but always on the CPU, then moved:
``cos``/``sin`` can differ by an ulp between devices, and bit-exact KV contents need the one
table everywhere.  ``forward`` keeps the reference signature and runs the CUDA kernel with the
cache write disabled.
"""
from __future__ import annotations

import torch
from torch import nn

from ... import ops


def build_cos_sin_cache(rotary_dim: int, max_position_embeddings: int, rope_theta: float) -> torch.Tensor:
    exponent = torch.arange(0, rotary_dim, 2, dtype=torch.float, device="cpu") / rotary_dim
    inv_freq = 1.0 / (rope_theta ** exponent)
    t = torch.arange(max_position_embeddings, dtype=torch.float, device="cpu")
    freqs = torch.einsum("i,j -> ij", t, inv_freq)
    return torch.cat((freqs.cos(), freqs.sin()), dim=-1)


class RotaryEmbedding(nn.Module):
    def __init__(self, rotary_dim: int, max_position_embeddings: int, rope_theta: float, device=None) -> None:
        super().__init__()
        self.rotary_dim = rotary_dim
        self.max_position_embeddings = max_position_embeddings
        self.rope_theta = rope_theta
        cache = build_cos_sin_cache(rotary_dim, max_position_embeddings, rope_theta)
        self.register_buffer("cos_sin_cache", cache.to(device) if device is not None else cache, persistent=False)

    def forward(self, positions: torch.Tensor, query: torch.Tensor, key: torch.Tensor):
        """Rotate ``query [T,Hq,D]`` and ``key [T,Hkv,D]`` in place and return them."""
        ops.rope_kv_write(query, key, key, positions, self.cos_sin_cache, None, None, None, k_in_place=True)
        return query, key
