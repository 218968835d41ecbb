"""Sampler: drop-in for ``minivllm/models/layers/sampler.py:9-31`` on the fused CUDA kernel.

``forward(logits, temperatures, top_p, top_k)`` keeps the reference's parameter order.  Without
top-k/top-p tensors the result is the greedy argmax of ``logits / temperature`` (the reference's
behaviour: temperature alone never randomises, ``sampler.py:31``).  With ``top_k`` the kernel
applies temperature, keeps each row's k largest logits and draws by Gumbel-max from a seeded
Philox stream.  ``top_p`` is accepted for signature parity; nucleus filtering is not implemented
and a request for it (any value < 1) raises.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from ... import ops


class Sampler(nn.Module):
    def __init__(self, seed: int = 0):
        super().__init__()
        self.seed = seed
        self.offset = 0            # advanced once per random draw so steps use fresh noise

    def forward(self, logits: torch.Tensor, temperatures: Optional[torch.Tensor] = None,
                top_p: Optional[torch.Tensor] = None, top_k: Optional[torch.Tensor] = None,
                scatter_table: Optional[torch.Tensor] = None, scatter_index: Optional[torch.Tensor] = None
                ) -> torch.Tensor:
        if logits.dtype != torch.bfloat16:
            logits = logits.to(torch.bfloat16)
        if top_p is not None and bool((top_p < 1.0).any()):
            raise NotImplementedError("top-p sampling is not implemented; use top_k")
        if top_k is None:
            return ops.sample(logits, temperatures, scatter_table=scatter_table, scatter_index=scatter_index)
        out = ops.sample(logits, temperatures, top_k, self.seed, self.offset, scatter_table=scatter_table,
                         scatter_index=scatter_index)
        self.offset += 1
        return out
