"""The packing <-> attention contract: one object per forward pass.

Field names, dtypes and meanings are those of ``minivllm/executor/context.py:5-81``:
``prefill`` (a step is all-prefill or all-decode), ``cu_seqlens_q/k`` int32 ``[B+1]``,
``max_seqlen_q/k`` host ints, ``positions`` int64 ``[T]``, ``slot_mapping`` int32 ``[T]`` (``-1``
= do not write), ``cache_seqlens`` int32 ``[B]`` (decode only; counts the new token),
``block_table`` int32 ``[B,W]`` right-padded with ``-1`` (``None`` for a prefill without cached
prefixes).

Two extras ride along for the CUDA kernels: the split-decode plan, which depends only on
``cache_seqlens`` and the window and is therefore made once per step and shared by all layers,
and a device status word the kernels report bad indices into.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch


@dataclass
class Context:
    prefill: bool = False
    cu_seqlens_q: Optional[torch.Tensor] = None
    cu_seqlens_k: Optional[torch.Tensor] = None
    max_seqlen_q: int = 0
    max_seqlen_k: int = 0
    positions: Optional[torch.Tensor] = None
    slot_mapping: Optional[torch.Tensor] = None
    cache_seqlens: Optional[torch.Tensor] = None
    block_table: Optional[torch.Tensor] = None
    # extension (mixed step): the last num_decode sequences of a prefill-shaped step hold one query token each
    # and are attended by the decode kernel; cache_seqlens then holds THEIR lengths
    num_decode: int = 0
    # extension: the prefill launch's work as a list, int32 [n, 2] of (sequence, query block) with the blocks that
    # see the most keys first, built on the host while packing (ops.build_prefill_items) for query blocks of
    # prefill_item_rows rows; the attention layer hands it to the kernel when its head layout uses that block size
    prefill_items: Optional[torch.Tensor] = field(default=None, repr=False, compare=False)
    prefill_item_rows: int = 0

    # filled by the attention layer on first use within this forward pass
    decode_plans: dict = field(default_factory=dict, repr=False, compare=False)
    # optional device int32[4]; kernels record out-of-range slots / block ids here
    status: Optional[torch.Tensor] = field(default=None, repr=False, compare=False)
