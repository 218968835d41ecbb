"""Varlen prefill and paged decode attention: gather through the block table, SDPA in fp32.

This is the definition the CUDA kernels are checked against.  It stands where
the reference calls ``flash_attn_varlen_func`` (``minivllm/models/layers/attention.py:84-87``)
and ``flash_attn_with_kvcache`` (``:90-91``), both from the absent third-party
``mini_flash_attention`` package: PARITY UNPINNED for the arithmetic itself.

Conventions (each follows a reference line):
* GQA head map ``kv = h // (Hq/Hkv)``; scale defaults to ``D**-0.5``
  (``qwen3.py:32``; ``gemma3.py:36`` with ``query_pre_attn_scalar == D``).
* causal mask is bottom-right aligned: query ``i`` of a sequence with
  ``q_len <= k_len`` sits at absolute position ``p = k_len - q_len + i`` and
  sees keys ``j <= p`` (matches ``positions = range(cached, n)``, ``executor.py:94``).
* sliding window ``(left, -1)``: key ``j`` visible iff ``p - left <= j <= p``
  (the layer's docstring, ``attention.py:56-60``); ``left < 0`` means no window.
* decode: one query per sequence at position ``cache_seqlens[b] - 1``
  (``executor.py:138-139``: the new token is counted and already written);
  rows with ``cache_seqlens == 0`` (graph padding, ``graph.py:68``) return zeros.
"""
from __future__ import annotations

import torch


def _sdpa(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
          q_pos0: int, window_left: int) -> torch.Tensor:
    """q ``[Tq,Hq,D]``, k/v ``[Tk,Hkv,D]`` of ONE sequence -> fp32 ``[Tq,Hq,D]``."""
    tq, hq, d = q.shape
    tk, hkv, _ = k.shape
    g = hq // hkv
    qf = q.float().transpose(0, 1)                                  # [Hq,Tq,D]
    kf = k.float().transpose(0, 1).repeat_interleave(g, dim=0)      # [Hq,Tk,D]
    vf = v.float().transpose(0, 1).repeat_interleave(g, dim=0)
    s = torch.matmul(qf, kf.transpose(1, 2)) * scale                # [Hq,Tq,Tk]
    p = torch.arange(q_pos0, q_pos0 + tq, device=q.device).unsqueeze(1)
    j = torch.arange(tk, device=q.device).unsqueeze(0)
    visible = j <= p
    if window_left >= 0:
        visible &= j >= p - window_left
    s = s.masked_fill(~visible.unsqueeze(0), float("-inf"))
    return torch.matmul(torch.softmax(s, dim=-1), vf).transpose(0, 1)


def gather_kv(cache: torch.Tensor, block_row: torch.Tensor, length: int) -> torch.Tensor:
    """Rows ``0..length-1`` of one sequence from ``cache [blocks,bs,Hkv,D]``."""
    bs = cache.shape[1]
    nblk = -(-length // bs)
    ids = block_row[:nblk].long()
    return cache[ids].reshape(nblk * bs, *cache.shape[2:])[:length]


def prefill(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
            cu_seqlens_q: torch.Tensor, cu_seqlens_k: torch.Tensor,
            block_table: torch.Tensor | None = None, scale: float | None = None,
            window_left: int = -1, out_dtype=None) -> torch.Tensor:
    """Causal varlen attention.

    Without ``block_table`` ``k``/``v`` are dense ``[T_k,Hkv,D]`` sliced by
    ``cu_seqlens_k``; with it they are the paged pool ``[blocks,bs,Hkv,D]`` and each
    sequence's keys ``0..k_len-1`` are gathered through its table row
    (the reference swaps in the pool at ``attention.py:82-83``).
    """
    d = q.shape[-1]
    scale = d ** -0.5 if scale is None else scale
    out = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
    cq, ck = cu_seqlens_q.tolist(), cu_seqlens_k.tolist()
    for s in range(len(cq) - 1):
        ql, kl = cq[s + 1] - cq[s], ck[s + 1] - ck[s]
        if ql == 0:
            continue
        if block_table is None:
            ks, vs = k[ck[s]:ck[s + 1]], v[ck[s]:ck[s + 1]]
        else:
            ks, vs = gather_kv(k, block_table[s], kl), gather_kv(v, block_table[s], kl)
        out[cq[s]:cq[s + 1]] = _sdpa(q[cq[s]:cq[s + 1]], ks, vs, scale, kl - ql, window_left)
    return out.to(out_dtype or q.dtype)


def decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
           cache_seqlens: torch.Tensor, block_table: torch.Tensor,
           scale: float | None = None, window_left: int = -1, out_dtype=None) -> torch.Tensor:
    """q ``[B,Hq,D]`` (one token per sequence) against ``cache_seqlens[b]`` cached keys."""
    d = q.shape[-1]
    scale = d ** -0.5 if scale is None else scale
    out = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
    for b, n in enumerate(cache_seqlens.tolist()):
        if n == 0:
            continue
        ks, vs = gather_kv(k_cache, block_table[b], n), gather_kv(v_cache, block_table[b], n)
        if window_left >= 0:                      # only the visible tail matters
            lo = max(0, n - 1 - window_left)
            out[b] = _sdpa(q[b:b + 1], ks[lo:], vs[lo:], scale, n - 1 - lo, -1)[0]
        else:
            out[b] = _sdpa(q[b:b + 1], ks, vs, scale, n - 1, -1)[0]
    return out.to(out_dtype or q.dtype)
