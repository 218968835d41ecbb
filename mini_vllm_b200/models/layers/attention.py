"""Attention layer: drop-in for ``FlashAttention`` of ``minivllm/models/layers/attention.py:46-92``.

Same constructor, same ``forward(ctx, q, k, v)`` contract (q/k already rotated; k/v are written
to the paged cache at ``ctx.slot_mapping`` first; prefill attends causally over ``cu_seqlens``,
decode attends one token per sequence over ``cache_seqlens`` through ``block_table``), same
``k_cache``/``v_cache`` attributes that the executor rebinds to views of its KV pool.
``forward_fused`` additionally takes ``positions`` and the cos/sin table and applies the rotary
embedding inside the KV-write kernel, saving one round trip of q and k through HBM.

Unlike the reference, ``scaling`` and ``sliding_window`` are honoured (the reference stores both
and passes neither to its attention calls, ``attention.py:84-91``).
"""
from __future__ import annotations

import torch
from torch import nn

from ... import ops
from ...executor.context import Context

_workspaces: dict = {}
_superseded: list = []      # outgrown buffers stay allocated: captured CUDA graphs keep writing through their pointers


def _decode_workspace(device, max_seqs: int, num_heads: int, head_dim: int, window_left: int) -> torch.Tensor:
    """One scratch buffer per (device, head shape, window); a larger one takes its place when a larger batch
    arrives.  The smaller buffer is never freed: a graph captured while it was current has its address
    baked in, and a replay after the memory went back to the allocator would scribble over someone else."""
    key = (device, num_heads, head_dim, window_left)
    ws = _workspaces.get(key)
    need = ops._cabi.load().mvb_decode_workspace_bytes(max_seqs, num_heads, head_dim)
    if ws is None or ws.numel() < need:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("decode workspace must be allocated before CUDA graph capture "
                               "(run one eager decode step of the largest batch first)")
        if ws is not None:
            _superseded.append(ws)
        ws = ops.decode_workspace(max(max_seqs, 512), num_heads, head_dim, device)
        _workspaces[key] = ws
    return ws


class FlashAttention(nn.Module):
    def __init__(self, num_heads: int, head_dim: int, scaling: float, num_kv_heads: int,
                 sliding_window=(-1, -1)):
        super().__init__()
        self.num_heads = num_heads
        self.head_dim = head_dim
        self.scaling = scaling
        self.num_kv_heads = num_kv_heads
        self.sliding_window = tuple(sliding_window)
        # placeholders the executor replaces with views of its KV pool (found by hasattr)
        self.k_cache = self.v_cache = torch.tensor([])
        self._item_rows = None            # query-block size of the prefill kernel's work items for this head layout

    @property
    def window_left(self) -> int:
        left = self.sliding_window[0]
        return int(left) if left is not None and left >= 0 else -1

    def _has_cache(self) -> bool:
        return self.k_cache.numel() > 0 and self.v_cache.numel() > 0

    def forward(self, ctx: Context, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        if self._has_cache():
            ops.rope_kv_write(None, k, v, None, None, ctx.slot_mapping, self.k_cache, self.v_cache,
                              k_in_place=False, status=ctx.status)
        return self._attend(ctx, q, k, v)

    def forward_fused(self, ctx: Context, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                      positions: torch.Tensor, cos_sin_cache: torch.Tensor) -> torch.Tensor:
        """q, k NOT yet rotated: RoPE (in place on q and k) + cache write in one kernel, then attention."""
        has_cache = self._has_cache()
        ops.rope_kv_write(q, k, v, positions, cos_sin_cache, ctx.slot_mapping if has_cache else None,
                          self.k_cache if has_cache else None, self.v_cache if has_cache else None,
                          k_in_place=ctx.prefill and ctx.block_table is None, status=ctx.status)
        return self._attend(ctx, q, k, v)

    def forward_fused_norm(self, ctx: Context, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                           positions: torch.Tensor, cos_sin_cache: torch.Tensor, q_weight: torch.Tensor,
                           k_weight: torch.Tensor, eps: float, unit_offset: bool) -> torch.Tensor:
        """q, k straight from the projection (views of the packed qkv output): per-head RMSNorm, RoPE
        and the cache write in one kernel (q and k updated in place), then attention."""
        has_cache = self._has_cache()
        ops.qk_norm_rope_kv_write(q, k, v, q_weight, k_weight, eps, unit_offset, positions, cos_sin_cache,
                                  ctx.slot_mapping if has_cache else None, self.k_cache if has_cache else None,
                                  self.v_cache if has_cache else None,
                                  k_in_place=ctx.prefill and ctx.block_table is None, status=ctx.status)
        return self._attend(ctx, q, k, v)

    def _items(self, ctx: Context):
        """The step's prefill work list, if the packing step built one for this layer's query-block size."""
        if ctx.prefill_items is None:
            return None
        if self._item_rows is None:
            self._item_rows = ops.prefill_item_rows(self.num_heads, self.num_kv_heads, self.head_dim)
        return ctx.prefill_items if ctx.prefill_item_rows == self._item_rows else None

    def _attend_mixed(self, ctx: Context, q: torch.Tensor) -> torch.Tensor:
        """A step holding both kinds of sequence (an extension; the reference's Context is one or the
        other): the prompts go through the prefill kernel, the single-token sequences at the end through
        the decode kernel, both over the paged pool the write kernel has just filled."""
        nd = ctx.num_decode
        bp, tp = ctx.cu_seqlens_q.numel() - 1 - nd, q.shape[0] - nd
        out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
        ops.prefill_attn(q[:tp], self.k_cache, self.v_cache, ctx.cu_seqlens_q[:bp + 1], ctx.cu_seqlens_k[:bp + 1],
                         ctx.max_seqlen_q, self.scaling, self.window_left, block_table=ctx.block_table[:bp],
                         out=out[:tp], status=ctx.status, items=self._items(ctx))
        wl = self.window_left
        table = ctx.block_table[bp:]
        ws = ctx.decode_plans.get(wl)
        if ws is None:
            ws = _decode_workspace(q.device, nd, self.num_heads, self.head_dim, wl)
            ops.decode_plan(ctx.cache_seqlens, wl, self.num_heads, self.num_kv_heads, self.head_dim, ws,
                            block_table=table, block_size=self.k_cache.shape[1])
            ctx.decode_plans[wl] = ws
        ops.decode_attn(q[tp:], self.k_cache, self.v_cache, ctx.cache_seqlens, table, self.scaling, wl, ws, out=out[tp:],
                        status=ctx.status)
        return out

    def _attend(self, ctx: Context, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        if ctx.prefill and ctx.num_decode:
            return self._attend_mixed(ctx, q)
        if ctx.prefill:
            if ctx.block_table is not None:        # prefix cache in play: keys come from the pool
                return ops.prefill_attn(q, self.k_cache, self.v_cache, ctx.cu_seqlens_q, ctx.cu_seqlens_k,
                                        ctx.max_seqlen_q, self.scaling, self.window_left,
                                        block_table=ctx.block_table, status=ctx.status, items=self._items(ctx))
            return ops.prefill_attn(q, k, v, ctx.cu_seqlens_q, ctx.cu_seqlens_k, ctx.max_seqlen_q, self.scaling,
                                    self.window_left, status=ctx.status, items=self._items(ctx))
        # decode: q [B,Hq,D] -> [B,1,Hq,D] like flash_attn_with_kvcache on q.unsqueeze(1)
        wl = self.window_left
        ws = ctx.decode_plans.get(wl)
        if ws is None:
            ws = _decode_workspace(q.device, ctx.cache_seqlens.numel(), self.num_heads, self.head_dim, wl)
            ops.decode_plan(ctx.cache_seqlens, wl, self.num_heads, self.num_kv_heads, self.head_dim, ws,
                            block_table=ctx.block_table, block_size=self.k_cache.shape[1])
            ctx.decode_plans[wl] = ws
        o = ops.decode_attn(q, self.k_cache, self.v_cache, ctx.cache_seqlens, ctx.block_table, self.scaling, wl, ws,
                            status=ctx.status)
        return o.unsqueeze(1)
