"""Sampler restated from ``minivllm/models/layers/sampler.py:9-31`` (CPU).

Greedy path (no top-k/top-p tensors): optional divide by temperature, then
``argmax`` with the lowest index winning ties — pinned bit-for-bit (CPU
``torch.argmax`` returns the first maximum).

Random path: the reference hands the logits to flashinfer with top-k and top-p
swapped (``executor.py:195`` vs ``sampler.py:9-13``) and without any seed, so it
has no reproducible output to pin.  The intended semantics are implemented
instead: temperature, keep every logit >= the k-th largest, keep the smallest most-likely set whose
softmax mass reaches top_p (ties with its last member included), then Gumbel-max
with a counter-based Philox4x32-10 stream keyed by (seed, offset, row, column).
"""
from __future__ import annotations

import numpy as np
import torch

_M0, _M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
_W0, _W1 = np.uint32(0x9E3779B9), np.uint32(0xBB67AE85)
_MASK = np.uint64(0xFFFFFFFF)


def philox4x32(counter: np.ndarray, key: np.ndarray) -> np.ndarray:
    """Philox4x32-10 (Salmon et al., SC'11).  counter ``[n,4]`` u32, key ``[n,2]`` u32 -> ``[n,4]`` u32."""
    c = counter.astype(np.uint32).copy()
    k = key.astype(np.uint32).copy()
    for _ in range(10):
        p0 = _M0 * c[:, 0].astype(np.uint64)
        p1 = _M1 * c[:, 2].astype(np.uint64)
        hi0, lo0 = (p0 >> np.uint64(32)).astype(np.uint32), (p0 & _MASK).astype(np.uint32)
        hi1, lo1 = (p1 >> np.uint64(32)).astype(np.uint32), (p1 & _MASK).astype(np.uint32)
        c = np.stack([hi1 ^ c[:, 1] ^ k[:, 0], lo1, hi0 ^ c[:, 3] ^ k[:, 1], lo0], axis=1)
        k = np.stack([k[:, 0] + _W0, k[:, 1] + _W1], axis=1)
    return c


def uniform_open(seed: int, offset: int, rows: int, cols: int) -> np.ndarray:
    """fp32 uniforms in (0,1): element (r,c) uses word ``c%4`` of Philox(counter=(c//4, r, offset_lo, offset_hi), key=seed)."""
    ngrp = -(-cols // 4)
    r = np.repeat(np.arange(rows, dtype=np.uint32), ngrp)
    gidx = np.tile(np.arange(ngrp, dtype=np.uint32), rows)
    ctr = np.stack([gidx, r,
                    np.full_like(r, offset & 0xFFFFFFFF), np.full_like(r, (offset >> 32) & 0xFFFFFFFF)], axis=1)
    key = np.stack([np.full_like(r, seed & 0xFFFFFFFF), np.full_like(r, (seed >> 32) & 0xFFFFFFFF)], axis=1)
    words = philox4x32(ctr, key).reshape(rows, ngrp * 4)[:, :cols]
    # 23 random bits, centred in their bucket (exact in fp32): never 0 and never 1
    return ((words >> np.uint32(9)).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 8388608.0)


def greedy(logits: torch.Tensor, temperatures: torch.Tensor | None = None) -> torch.Tensor:
    if temperatures is not None:
        logits = logits / temperatures.unsqueeze(-1)          # sampler.py:15-16
    return torch.argmax(logits, dim=-1)                       # sampler.py:31


def gumbel_scores(logits: torch.Tensor, temperatures: torch.Tensor | None,
                  top_k: torch.Tensor | None, seed: int, offset: int,
                  top_p: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 ``[B,V]`` perturbed scores; entries outside the top-k / top-p set are -inf."""
    x = logits.float()
    if temperatures is not None:
        x = x / temperatures.float().unsqueeze(-1)
    b, v = x.shape
    if top_k is not None:
        for r, k in enumerate(top_k.tolist()):
            if 0 < k < v:
                kth = torch.topk(x[r], k).values[-1]
                x[r] = torch.where(x[r] >= kth, x[r], torch.full_like(x[r], float("-inf")))
    if top_p is not None:
        for r, pr in enumerate(top_p.tolist()):
            if pr < 1.0:
                keep = torch.isfinite(x[r])
                probs = torch.softmax(x[r].double(), dim=-1)
                order = torch.argsort(probs, descending=True, stable=True)
                csum = torch.cumsum(probs[order], 0)
                n_keep = int(torch.searchsorted(csum, torch.tensor(pr * float(csum[-1]), dtype=torch.float64))) + 1
                cut = x[r][order[min(n_keep, v) - 1]]            # ties with the last kept token stay
                x[r] = torch.where((x[r] >= cut) & keep, x[r], torch.full_like(x[r], float("-inf")))
    u = torch.from_numpy(uniform_open(seed, offset, b, v))
    return x - torch.log(-torch.log(u))


def sample(logits, temperatures, top_k, seed: int, offset: int) -> torch.Tensor:
    return torch.argmax(gumbel_scores(logits, temperatures, top_k, seed, offset), dim=-1)
