"""Shared builders for the parity tests (CPU tensors; tests copy them to the device)."""
from __future__ import annotations

import torch

from mini_vllm_b200.workloads import BLOCK_SIZE, cdiv, generator, randn_bf16, table_tensor  # noqa: F401

ATTN_MAX_ABS = 2e-2     # tolerance of the attention outputs against the fp32 oracle (bf16 inputs)
ATTN_MEAN_ABS = 2e-3


def poison_pool(num_blocks: int, hkv: int, d: int, block_size: int = BLOCK_SIZE) -> torch.Tensor:
    """A KV pool whose every element is a bf16 NaN: any read of an unwritten slot shows up."""
    return torch.full((num_blocks, block_size, hkv, d), float("nan"), dtype=torch.bfloat16)


def fill_paged(g: torch.Generator, lens: list[int], tables: list[list[int]], num_blocks: int, hkv: int, d: int,
               block_size: int = BLOCK_SIZE):
    """Random K/V for every sequence, scattered into NaN-poisoned pools through the block tables."""
    k_pool, v_pool = poison_pool(num_blocks, hkv, d, block_size), poison_pool(num_blocks, hkv, d, block_size)
    for n, blocks in zip(lens, tables):
        k, v = randn_bf16(g, n, hkv, d), randn_bf16(g, n, hkv, d)
        for i, blk in enumerate(blocks):
            lo, hi = i * block_size, min(n, (i + 1) * block_size)
            if lo >= hi:
                break
            k_pool[blk, :hi - lo] = k[lo:hi]
            v_pool[blk, :hi - lo] = v[lo:hi]
    return k_pool, v_pool


def sequential_tables(g: torch.Generator, lens: list[int], num_blocks: int, block_size: int = BLOCK_SIZE):
    perm = torch.randperm(num_blocks, generator=g).tolist()
    out, cur = [], 0
    for n in lens:
        nb = max(1, cdiv(n, block_size))
        out.append(perm[cur:cur + nb])
        cur += nb
    assert cur <= num_blocks
    return out


def assert_close_attn(got: torch.Tensor, want: torch.Tensor, what: str = "") -> None:
    got, want = got.float().cpu(), want.float().cpu()
    assert torch.isfinite(got).all(), f"{what}: non-finite output"
    err = (got - want).abs()
    assert err.max().item() <= ATTN_MAX_ABS, f"{what}: max-abs {err.max().item():.4g}"
    assert err.mean().item() <= ATTN_MEAN_ABS, f"{what}: mean-abs {err.mean().item():.4g}"
