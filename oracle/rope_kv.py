"""RoPE and KV-cache write restated from the reference layers (PyTorch eager, CPU).

RoPE follows ``minivllm/models/layers/rotary.py``: table :32-47, apply :6-14,
gather and broadcast :59-71.  The reference wraps ``forward`` in
``torch.compile``; the oracle is the eager arithmetic (each product and the
sum/difference rounded separately in fp32, one final rounding to bf16).
KV write follows ``minivllm/models/layers/attention.py:13-43``.
"""
from __future__ import annotations

import torch


def cos_sin_table(rotary_dim: int, max_pos: int, theta: float) -> torch.Tensor:
    """fp32 ``[max_pos, rotary_dim]`` = cat(cos, sin) (rotary.py:32-47)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float) / rotary_dim))
    t = torch.arange(max_pos, dtype=torch.float)
    freqs = torch.einsum("i,j -> ij", t, inv_freq)
    return torch.cat((freqs.cos(), freqs.sin()), dim=-1)


def rotate(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half (non-interleaved) in fp32, cast back (rotary.py:6-14)."""
    x1, x2 = torch.chunk(x.float(), 2, dim=-1)
    y1 = x1 * cos - x2 * sin
    y2 = x2 * cos + x1 * sin
    return torch.cat((y1, y2), dim=-1).to(x.dtype)


def apply_rope(positions: torch.Tensor, q: torch.Tensor, k: torch.Tensor,
               table: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """q ``[T,Hq,D]``, k ``[T,Hkv,D]``; the same cos/sin row for every head (rotary.py:59-71)."""
    cos, sin = table[positions].chunk(2, dim=-1)
    cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    return rotate(q, cos, sin), rotate(k, cos, sin)


def store_kvcache(key: torch.Tensor, value: torch.Tensor, k_cache: torch.Tensor,
                  v_cache: torch.Tensor, slot_mapping: torch.Tensor) -> None:
    """Row ``i`` goes to flat cache row ``slot[i]``; ``slot == -1`` is skipped (attention.py:24-33)."""
    n, h, d = key.shape
    keep = slot_mapping >= 0
    idx = slot_mapping[keep].long()
    k_cache.view(-1, h * d).index_copy_(0, idx, key.reshape(n, h * d)[keep])
    v_cache.view(-1, h * d).index_copy_(0, idx, value.reshape(n, h * d)[keep])


def qk_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, unit_offset: bool) -> torch.Tensor:
    """Per-head RMSNorm as the models apply it before RoPE: ``nn.RMSNorm`` (qwen3.py:64-65,89-90) or
    Gemma's fp32 ``(1 + w)`` form (gemma3.py:12-24,97-98)."""
    if not unit_offset:
        return torch.nn.functional.rms_norm(x, (x.shape[-1],), weight, eps)
    xf = x.float()
    xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (xf * (1.0 + weight.float())).type_as(x)
