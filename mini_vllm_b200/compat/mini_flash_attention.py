"""``mini_flash_attention`` as the reference imports it, backed by ``mvb_prefill_attn`` / ``mvb_decode_attn``.

The reference binds its attention with
``from mini_flash_attention import flash_attn_with_kvcache, flash_attn_varlen_func``
(``minivllm/models/layers/attention.py:7``) and calls

    flash_attn_varlen_func(q, k, v, max_seqlen_q=, cu_seqlens_q=, max_seqlen_k=, cu_seqlens_k=, causal=True)   (:84-87)
    flash_attn_with_kvcache(q.unsqueeze(1), k_cache, v_cache, cache_seqlens=, block_table=)                     (:90-91)

Both are provided here with exactly those keywords (plus the optional ``softmax_scale``, ``window_size`` and
``block_table`` that the interchangeable flash_attn functions take), so an unmodified reference checkout runs on
the CUDA kernels after ``mini_vllm_b200.compat.install()``.

One call of the reference cannot work through this seam: with a cached prefix it passes the 4-D paged pool as
``k``/``v`` but no block table (``attention.py:82-87``), and without the table there is no way to tell which
blocks a sequence owns.  That call raises here with a message that says so; ``FlashAttention`` of this package
passes ``ctx.block_table`` instead.
"""
from __future__ import annotations

import torch

from .. import ops

_workspaces: dict = {}
_superseded: list = []


def _workspace(device, rows: int, num_heads: int, head_dim: int) -> torch.Tensor:
    key = (device, num_heads, head_dim)
    ws = _workspaces.get(key)
    need = ops._cabi.load().mvb_decode_workspace_bytes(rows, num_heads, head_dim)
    if ws is None or ws.numel() < need:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("the decode workspace must exist before CUDA graph capture: run the model once eagerly")
        if ws is not None:
            _superseded.append(ws)                   # a captured graph may still write through the old pointer
        ws = ops.decode_workspace(max(rows, 512), num_heads, head_dim, device)
        _workspaces[key] = ws
    return ws


def _window_left(window_size, causal: bool) -> int:
    left, right = window_size
    if not causal or (right is not None and right > 0):
        raise NotImplementedError("only causal attention is implemented (the reference passes causal=True)")
    return int(left) if left is not None and left >= 0 else -1


def flash_attn_varlen_func(q, k, v, cu_seqlens_q=None, cu_seqlens_k=None, max_seqlen_q=None, max_seqlen_k=None,
                           dropout_p: float = 0.0, softmax_scale=None, causal: bool = False,
                           window_size=(-1, -1), block_table=None, **unsupported):
    """Causal varlen attention: ``q [T_q,H_q,D]``; ``k``/``v`` dense ``[T_k,H_kv,D]`` or, with ``block_table``
    ``[B,W]``, the paged pool ``[blocks,block_size,H_kv,D]``.  Returns ``[T_q,H_q,D]``."""
    if unsupported:
        raise TypeError(f"unsupported arguments: {sorted(unsupported)}")
    if dropout_p:
        raise NotImplementedError("dropout is not implemented")
    if cu_seqlens_q is None or cu_seqlens_k is None or max_seqlen_q is None:
        raise TypeError("cu_seqlens_q, cu_seqlens_k and max_seqlen_q are required")
    if k.dim() == 4 and block_table is None:
        raise ValueError("k and v are a paged pool [blocks, block_size, heads, head_dim] but no block_table was given: "
                         "the reference's prefix-cached prefill (attention.py:82-87) does not pass one, so that branch "
                         "cannot go through this function; pass block_table=ctx.block_table")
    scale = q.shape[-1] ** -0.5 if softmax_scale is None else float(softmax_scale)
    return ops.prefill_attn(q, k, v, cu_seqlens_q, cu_seqlens_k, int(max_seqlen_q), scale,
                            _window_left(window_size, causal), block_table=block_table)


def flash_attn_with_kvcache(q, k_cache, v_cache, k=None, v=None, cache_seqlens=None, block_table=None,
                            softmax_scale=None, causal: bool = True, window_size=(-1, -1), **unsupported):
    """One query token per sequence against the paged cache: ``q [B,1,H_q,D]`` -> ``[B,1,H_q,D]``."""
    if unsupported:
        raise TypeError(f"unsupported arguments: {sorted(unsupported)}")
    if k is not None or v is not None:
        raise NotImplementedError("appending k/v inside the call is not implemented: write the cache first")
    if cache_seqlens is None or block_table is None:
        raise TypeError("cache_seqlens and block_table are required (the cache is paged)")
    if q.dim() != 4 or q.shape[1] != 1:
        raise ValueError("q must be [batch, 1, heads, head_dim]")
    q3 = q[:, 0]
    rows, hq, d = q3.shape
    hkv = k_cache.shape[2]
    wl = _window_left(window_size, True)
    scale = d ** -0.5 if softmax_scale is None else float(softmax_scale)
    ws = _workspace(q.device, rows, hq, d)
    ops.decode_plan(cache_seqlens, wl, hq, hkv, d, ws, block_table=block_table, block_size=k_cache.shape[1])
    return ops.decode_attn(q3, k_cache, v_cache, cache_seqlens, block_table, scale, wl, ws).unsqueeze(1)
