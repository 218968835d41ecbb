"""CUDA-graph replay of the decode step.

Same scheme as ``minivllm/executor/graph.py``: static input buffers sized for
``min(max_num_batched_seqs, 256)`` rows, one graph per batch size in
``[1, 2, 4, 8, 16, 32, ...]`` captured largest-first into one memory pool, replay on the
smallest captured size that fits.  The difference is how the static buffers get filled: the
executor's decode packing kernel writes them directly (including the padding rows: slot -1,
length 0), so ``replay`` launches no staging copies when the context already aliases them.
A context built elsewhere is still accepted and copied in, as the reference does.
"""
from __future__ import annotations

import torch

from ..ops import LaunchCounter
from .context import Context


class CudaGraphRunner:
    def __init__(self, model, config, max_batch_size: int, status: torch.Tensor | None = None):
        self.model = model
        self.config = config
        self.max_batch_size = min(max_batch_size, getattr(config, "max_graph_batch_size", 256))
        sizes = [b for b in (1, 2, 4, 8) if b <= self.max_batch_size] + list(range(16, self.max_batch_size + 1, 16))
        self.batch_size_list = sorted(set(sizes + [self.max_batch_size]))   # the largest batch always has a graph
        self.graphs: dict[int, torch.cuda.CUDAGraph] = {}
        self.launches: dict[int, int] = {}       # library kernels inside each captured graph
        self.pool = None
        self.status = status
        dev, m = torch.device("cuda", torch.cuda.current_device()), self.max_batch_size
        self.input_ids = torch.zeros(m, dtype=torch.int64, device=dev)
        self.positions = torch.zeros(m, dtype=torch.int64, device=dev)
        self.slot_mapping = torch.full((m,), -1, dtype=torch.int32, device=dev)
        self.cache_seqlens = torch.zeros(m, dtype=torch.int32, device=dev)
        self.block_table = torch.full((m, config.kv_cache_num_blocks), -1, dtype=torch.int32, device=dev)
        # The captured step ends at the rows the lm_head reads (final norm applied); the head itself - the GEMM and
        # the sampler, or the fused argmax kernel - runs behind the replay, where the executor knows whether the
        # batch samples greedily.  (The reference captures the logits, graph.py:21.)
        self.outputs = torch.zeros(m, config.hf_config.hidden_size, dtype=config.hf_config.dtype, device=dev)

    def padded_size(self, bs: int) -> int:
        return next(b for b in self.batch_size_list if b >= bs)

    def static_context(self, batch_size: int) -> Context:
        return Context(prefill=False, positions=self.positions[:batch_size],
                       slot_mapping=self.slot_mapping[:batch_size], cache_seqlens=self.cache_seqlens[:batch_size],
                       block_table=self.block_table[:batch_size], status=self.status)

    @torch.inference_mode()
    def capture(self) -> None:
        for bs in reversed(self.batch_size_list):
            self._capture_batch(bs)

    def _capture_batch(self, bs: int) -> None:
        # one eager run first: lazy initialisation (cuBLAS handles, kernel attributes, the decode
        # workspace) must not happen inside the capture
        self.outputs[:bs] = self.model(self.static_context(bs), self.input_ids[:bs], self.positions[:bs], head=False)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        before = LaunchCounter.total
        with torch.cuda.graph(g, pool=self.pool):
            self.outputs[:bs] = self.model(self.static_context(bs), self.input_ids[:bs], self.positions[:bs], head=False)
        self.launches[bs] = LaunchCounter.total - before
        self.pool = g.pool()
        self.graphs[bs] = g
        torch.cuda.synchronize()

    def owns(self, ctx: Context) -> bool:
        return ctx.positions is not None and ctx.positions.data_ptr() == self.positions.data_ptr()

    @torch.inference_mode()
    def replay(self, ctx: Context, input_ids: torch.Tensor) -> torch.Tensor:
        """Runs the captured step; returns the ``[bs, hidden]`` rows for the head."""
        bs = input_ids.size(0)
        if not self.owns(ctx):                       # foreign context: stage it like graph.py:64-70
            self.input_ids[:bs] = input_ids
            self.positions[:bs] = ctx.positions
            self.slot_mapping.fill_(-1)
            self.slot_mapping[:bs] = ctx.slot_mapping
            self.cache_seqlens.zero_()
            self.cache_seqlens[:bs] = ctx.cache_seqlens
            self.block_table[:bs, :ctx.block_table.size(1)] = ctx.block_table
        padded = self.padded_size(bs)
        self.graphs[padded].replay()
        LaunchCounter.add(self.launches[padded])
        return self.outputs[:bs]
