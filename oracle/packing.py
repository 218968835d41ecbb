"""Batch packing restated from the reference executor (numpy, host only).

Follows ``minivllm/executor/executor.py``:
``_build_prefill_input`` :81-127, ``_build_decode_input`` :130-153,
``_build_block_table`` :156-163.  Inputs are per-sequence facts, the same ones
the reference reads off its ``Request`` objects (``tokens``, ``blocks``,
``num_cached_tokens``).
"""
from __future__ import annotations

import numpy as np


def build_block_table(blocks: list[list[int]]) -> np.ndarray:
    """Rows right-padded with -1 to the longest row, int32 (executor.py:156-163)."""
    width = max(len(b) for b in blocks)
    out = np.full((len(blocks), width), -1, dtype=np.int32)
    for i, b in enumerate(blocks):
        out[i, :len(b)] = b
    return out


def build_prefill_input(tokens: list[list[int]], blocks: list[list[int]],
                        cached: list[int], block_size: int) -> dict:
    """executor.py:81-127.  Returns numpy arrays plus the two host ints."""
    input_ids, positions, slots = [], [], []
    cu_q, cu_k = [0], [0]
    max_q = max_k = 0
    for toks, blks, c in zip(tokens, blocks, cached):
        n = len(toks)
        input_ids.append(np.asarray(toks[c:], dtype=np.int64))
        positions.append(np.arange(c, n, dtype=np.int64))
        cu_q.append(cu_q[-1] + n - c)
        cu_k.append(cu_k[-1] + n)
        max_q, max_k = max(max_q, n - c), max(max_k, n)
        # executor.py:102-111: slots for blocks c/bs .. last; the last block holds
        # n - (nblk-1)*bs tokens.  Warm-up requests carry no blocks and yield none.
        for i in range(c // block_size, len(blks)):
            start = blks[i] * block_size
            fill = block_size if i != len(blks) - 1 else n - (len(blks) - 1) * block_size
            slots.append(np.arange(start, start + fill, dtype=np.int32))
    cat = lambda xs, dt: np.concatenate(xs).astype(dt) if xs else np.zeros(0, dt)
    out = {
        "input_ids": cat(input_ids, np.int64),
        "positions": cat(positions, np.int64),
        "slot_mapping": cat(slots, np.int32),
        "cu_seqlens_q": np.asarray(cu_q, dtype=np.int32),
        "cu_seqlens_k": np.asarray(cu_k, dtype=np.int32),
        "max_seqlen_q": max_q,
        "max_seqlen_k": max_k,
        "block_table": None,
    }
    if cu_k[-1] > cu_q[-1]:                     # executor.py:113-114
        out["block_table"] = build_block_table(blocks)
    return out


def build_decode_input(tokens: list[list[int]], blocks: list[list[int]], block_size: int) -> dict:
    """executor.py:130-153: last token, its position, its slot, context length."""
    ids = np.asarray([t[-1] for t in tokens], dtype=np.int64)
    n = np.asarray([len(t) for t in tokens], dtype=np.int64)
    last_blk = np.asarray([b[-1] for b in blocks], dtype=np.int64)
    nblk = np.asarray([len(b) for b in blocks], dtype=np.int64)
    slot = last_blk * block_size + (n - (nblk - 1) * block_size) - 1
    return {
        "input_ids": ids,
        "positions": (n - 1).astype(np.int64),
        "slot_mapping": slot.astype(np.int32),
        "cache_seqlens": n.astype(np.int32),
        "block_table": build_block_table(blocks),
    }
