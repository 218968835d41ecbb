"""Seeded synthetic inputs for the ragged attention path.

Every generator follows one RNG convention so that "seed 0" means the same
bytes everywhere (tests, bench, oracle): a CPU ``torch.Generator``; integers via
``torch.randint(lo, hi + 1)``; permutations via ``torch.randperm``; normals via
``torch.randn(fp32).to(bf16)``; draw order is lengths, then the block
permutation, then q, k, v.  Tensors are always created on the CPU and copied.

The shapes are those of Qwen3-0.6B (16 q heads, 8 kv heads, head_dim 128) and
Gemma3-1B (4 q heads, 1 kv head, head_dim 256) with 256-token KV blocks.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

BLOCK_SIZE = 256


@dataclass(frozen=True)
class AttnShape:
    num_q_heads: int
    num_kv_heads: int
    head_dim: int
    num_layers: int = 1
    rope_theta: float = 1e6

    @property
    def group(self) -> int:
        return self.num_q_heads // self.num_kv_heads

    @property
    def kv_row_bytes(self) -> int:
        """Bytes of K plus V for one token in one layer (bf16)."""
        return 2 * self.num_kv_heads * self.head_dim * 2


QWEN3_0P6B = AttnShape(16, 8, 128, num_layers=28, rope_theta=1e6)
GEMMA3_1B = AttnShape(4, 1, 256, num_layers=26, rope_theta=1e6)


def generator(seed: int) -> torch.Generator:
    return torch.Generator(device="cpu").manual_seed(seed)


def randint(g: torch.Generator, lo: int, hi: int, n: int) -> list[int]:
    """n integers uniform in the closed range [lo, hi]."""
    return torch.randint(lo, hi + 1, (n,), generator=g).tolist()


def randn_bf16(g: torch.Generator, *shape: int) -> torch.Tensor:
    return torch.randn(*shape, generator=g, dtype=torch.float32).to(torch.bfloat16)


def log_uniform(g: torch.Generator, lo: int, hi: int, n: int) -> list[int]:
    u = torch.rand(n, generator=g, dtype=torch.float64)
    x = torch.exp(math.log(lo) + u * (math.log(hi) - math.log(lo)))
    return [min(hi, max(lo, int(v))) for v in x.tolist()]


def cdiv(a: int, b: int) -> int:
    return -(-a // b)


def assign_blocks(g: torch.Generator, lengths: list[int], pool_blocks: int,
                  reserve_tokens: int = 0) -> list[list[int]]:
    """Hand each sequence the next ids of a seeded permutation of the pool.

    ``reserve_tokens`` extra tokens per sequence are budgeted so that later
    decode steps never need a new block.
    """
    perm = torch.randperm(pool_blocks, generator=g).tolist()
    tables, cursor = [], 0
    for n in lengths:
        nb = cdiv(n + reserve_tokens, BLOCK_SIZE)
        if cursor + nb > pool_blocks:
            raise ValueError("KV pool too small for the workload")
        tables.append(perm[cursor:cursor + nb])
        cursor += nb
    return tables


def table_tensor(tables: list[list[int]], width: int | None = None, pad: int = -1) -> torch.Tensor:
    """Block lists -> int32 ``[B, W]`` right-padded with ``pad`` (the Context block-table layout)."""
    width = width or max(1, max(len(t) for t in tables))
    out = torch.full((len(tables), width), pad, dtype=torch.int32)
    for i, t in enumerate(tables):
        if t:
            out[i, :len(t)] = torch.tensor(t, dtype=torch.int32)
    return out


@dataclass
class SingleLayerCase:
    """One attention layer's worth of ragged work (configs 1, 3, 4)."""
    shape: AttnShape
    pool_blocks: int
    # prefill part (may be empty)
    prefill_lens: list[int] = field(default_factory=list)      # full k lengths
    prefill_cached: list[int] = field(default_factory=list)    # cached prefix lengths
    prefill_blocks: list[list[int]] = field(default_factory=list)
    # decode part (may be empty)
    decode_ctx: list[int] = field(default_factory=list)        # context incl. the new token
    decode_blocks: list[list[int]] = field(default_factory=list)
    window_left: int = -1


def config1(seed: int = 0, decode_steps: int = 32) -> tuple[SingleLayerCase, torch.Generator]:
    """8 sequences, prompt lengths U[16,512], 64-block pool, Qwen3 shapes."""
    g = generator(seed)
    lens = randint(g, 16, 512, 8)
    blocks = assign_blocks(g, lens, 64, reserve_tokens=decode_steps)
    case = SingleLayerCase(QWEN3_0P6B, 64, prefill_lens=lens, prefill_cached=[0] * 8,
                           prefill_blocks=blocks)
    return case, g


def config3(seed: int = 0, pool_blocks: int = 2200) -> tuple[SingleLayerCase, torch.Generator]:
    """16 prefills (half sharing a cached 512-token prefix) + 240 decodes, Qwen3 shapes."""
    g = generator(seed)
    suffix = randint(g, 100, 2048, 16)
    ctx = randint(g, 128, 4096, 240)
    perm = torch.randperm(pool_blocks, generator=g).tolist()
    cursor = 0

    def take(n: int) -> list[int]:
        nonlocal cursor
        if cursor + n > pool_blocks:
            raise ValueError("KV pool too small for the workload")
        out = perm[cursor:cursor + n]
        cursor += n
        return out

    shared = take(2)                                  # the resident 512-token prefix
    p_lens, p_cached, p_blocks = [], [], []
    for i, s in enumerate(suffix):
        if i % 2 == 0:
            p_lens.append(512 + s)
            p_cached.append(512)
            p_blocks.append(shared + take(cdiv(512 + s, BLOCK_SIZE) - 2))
        else:
            p_lens.append(s)
            p_cached.append(0)
            p_blocks.append(take(cdiv(s, BLOCK_SIZE)))
    d_blocks = [take(cdiv(c, BLOCK_SIZE)) for c in ctx]
    case = SingleLayerCase(QWEN3_0P6B, pool_blocks, prefill_lens=p_lens, prefill_cached=p_cached,
                           prefill_blocks=p_blocks, decode_ctx=ctx, decode_blocks=d_blocks)
    return case, g


def config4(seed: int = 0, pool_blocks: int = 1300, window_left: int = -1
            ) -> tuple[SingleLayerCase, torch.Generator]:
    """128 decodes with contexts U[512,4096], Gemma3-1B shapes; window 512 on local layers."""
    g = generator(seed)
    ctx = randint(g, 512, 4096, 128)
    blocks = assign_blocks(g, ctx, pool_blocks)
    case = SingleLayerCase(GEMMA3_1B, pool_blocks, decode_ctx=ctx, decode_blocks=blocks,
                           window_left=window_left)
    return case, g


def decode_kv_bytes(shape: AttnShape, ctx: list[int], window_left: int = -1) -> int:
    """Algorithmic K+V bytes one decode-attention launch must read (one layer)."""
    if window_left >= 0:
        ctx = [min(c, window_left + 1) for c in ctx]
    return sum(ctx) * shape.kv_row_bytes


def prefill_pairs(lens: list[int], cached: list[int], window_left: int = -1) -> int:
    """Number of (query, key) pairs a causal varlen prefill evaluates."""
    total = 0
    for n, c in zip(lens, cached):
        q = n - c
        if window_left < 0:
            total += q * c + q * (q + 1) // 2
        else:
            for p in range(c, n):
                total += min(p, window_left) + 1
    return total


def prefill_flops(shape: AttnShape, lens: list[int], cached: list[int], window_left: int = -1) -> int:
    return 4 * shape.num_q_heads * shape.head_dim * prefill_pairs(lens, cached, window_left)


@dataclass
class GenRequest:
    prompt: list[int]
    max_tokens: int


def config2_requests(seed: int = 0, n: int = 64, vocab: int = 151936) -> list[GenRequest]:
    """64 requests, prompt U[100,1024], output U[100,1024] capped so total <= 1024."""
    g = generator(seed)
    p_lens = randint(g, 100, 1024, n)
    o_lens = randint(g, 100, 1024, n)
    reqs = []
    for p, o in zip(p_lens, o_lens):
        p = min(p, 1023)                    # leave room for at least one generated token
        o = min(o, 1024 - p)
        toks = torch.randint(0, vocab, (p,), generator=g).tolist()
        reqs.append(GenRequest(toks, o))
    return reqs


def config5_requests(seed: int = 0, n: int = 4096, vocab: int = 151936) -> list[GenRequest]:
    """Prompt lengths log-uniform [32,4096], output lengths U[64,1024]."""
    g = generator(seed)
    p_lens = log_uniform(g, 32, 4096, n)
    o_lens = randint(g, 64, 1024, n)
    reqs = []
    for p, o in zip(p_lens, o_lens):
        toks = torch.randint(0, vocab, (p,), generator=g).tolist()
        reqs.append(GenRequest(toks, o))
    return reqs
