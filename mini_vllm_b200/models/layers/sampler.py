"""Sampler: drop-in for ``minivllm/models/layers/sampler.py:9-31`` on the fused CUDA kernel.

``forward(logits, temperatures, top_p, top_k)`` keeps the reference's parameter order.  Without
top-k/top-p tensors the result is the greedy argmax of ``logits / temperature`` (the reference's
behaviour: temperature alone never randomises, ``sampler.py:31``).  With ``top_k`` the kernel
applies temperature, keeps each row's k largest logits, then the nucleus of probability mass
``top_p`` among them, and draws by Gumbel-max from a seeded Philox stream (the reference hands both
to flashinfer, swapped and unseeded, ``executor.py:195`` vs ``sampler.py:9-13``).
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
        if top_k is None and top_p is None:
            return ops.sample(logits, temperatures, scatter_table=scatter_table, scatter_index=scatter_index)
        out = ops.sample(logits, temperatures, top_k, self.seed, self.offset, top_p=top_p,
                         scatter_table=scatter_table, scatter_index=scatter_index)
        self.offset += 1
        return out
