"""Executor: model, KV pool, device-side batch packing, CUDA-graph decode, sampling.

Counterpart of ``minivllm/executor/executor.py``.  The contract of ``_build_prefill_input`` /
``_build_decode_input`` / ``_build_block_table`` (``:81-163``) is unchanged — same tensors, dtypes
and shapes inside the same ``Context`` — but the per-token Python loops and the five pinned
uploads per step are gone: the host gathers per-SEQUENCE facts (lengths, cached lengths, block
lists, the new tokens) into one pinned int32 buffer with numpy, uploads it with a single copy, and
a packing kernel expands it on the device.
"""
from __future__ import annotations

import itertools
import logging

import numpy as np
import torch

from .. import ops
from ..engine.request import Request
from ..models.layers.sampler import Sampler
from ..models.loader import load_model
from ..scheduler.batch import Batch
from .context import Context
from .graph import CudaGraphRunner

log = logging.getLogger(__name__)


class _Staging:
    """A pinned host int32 buffer and its device twin, grown on demand; one upload per step."""

    def __init__(self, device):
        self.device = device
        self.host = torch.empty(0, dtype=torch.int32)
        self.dev = torch.empty(0, dtype=torch.int32, device=device)

    def upload(self, parts: list[np.ndarray]) -> torch.Tensor:
        n = sum(p.size for p in parts)
        if self.host.numel() < n:
            cap = max(n, 2 * self.host.numel(), 1 << 16)
            self.host = torch.empty(cap, dtype=torch.int32).pin_memory()
            self.dev = torch.empty(cap, dtype=torch.int32, device=self.device)
        view, cur = self.host.numpy(), 0
        for p in parts:
            view[cur:cur + p.size] = p
            cur += p.size
        self.dev[:n].copy_(self.host[:n], non_blocking=True)
        return self.dev[:n]


class Executor:
    RING = 4          # staging / result buffers in flight; the pipelined engine runs at most RING - 2 steps ahead

    @property
    def _stage(self) -> _Staging:
        return self._stages[self._step % self.RING]

    def __init__(self, config):
        self.config = config
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.block_size = config.kv_cache_block_size
        self.model = load_model(config, self.device)
        self.sampler = Sampler(seed=config.seed)
        self.status = ops.new_status(self.device)
        # a ring of staging buffers: with the pipelined engine the host prepares step k+1 while the
        # upload of step k may not have run yet
        self._stages = [_Staging(self.device) for _ in range(self.RING)]
        self._step = 0
        self.token_table = torch.zeros(0, dtype=torch.int64, device=self.device)   # last token per request slot
        self._out_ring = torch.zeros(self.RING, max(config.max_num_batched_seqs, 1), dtype=torch.int64).pin_memory()
        self.fused_head = bool(getattr(config, "fused_greedy_head", True))
        self.fused_head_max_rows = int(getattr(config, "fused_head_max_rows", 256))
        self._head_scratch = ops.lm_head_argmax_scratch(max(self.fused_head_max_rows, 16), self.device)
        hf = config.hf_config
        try:                                   # query-block size of the prefill kernel's work items for this model
            self.item_rows = ops.prefill_item_rows(hf.num_attention_heads, hf.num_key_value_heads, hf.head_dim)
        except Exception:
            self.item_rows = 0                 # (a head layout the kernel does not take: no list, the plain grid)
        self.h2d_bytes = 0                   # bytes uploaded by the packing path (for the bench's e2e line)
        self.d2h_bytes = 0
        self.graph_runner = None
        self._warmup_model()
        self._init_kv_cache()
        if config.use_cuda_graph:
            log.info("capturing CUDA graphs for decode")
            self.graph_runner = CudaGraphRunner(self.model, config, config.max_num_batched_seqs, self.status)
            self.graph_runner.capture()

    # ---- bring-up --------------------------------------------------------------------------------
    def _warmup_model(self) -> None:
        """A prefill of block-less zero-token requests before the KV pool exists (executor.py:62-78)."""
        torch.cuda.empty_cache()
        torch.cuda.reset_peak_memory_stats()
        self.execute(Batch(Batch.PREFILL, [Request([0] * 64) for _ in range(10)]))
        torch.cuda.empty_cache()

    def _init_kv_cache(self) -> None:
        """Pool ``[2, layers, blocks, block_size, kv_heads, head_dim]``; layer l's K is ``[0, l]`` (executor.py:31-60)."""
        cfg, hf = self.config, self.config.hf_config
        free, total = torch.cuda.mem_get_info()
        stats = torch.cuda.memory_stats()
        peak, current = stats["allocated_bytes.all.peak"], stats["allocated_bytes.all.current"]
        head_dim = getattr(hf, "head_dim", hf.hidden_size // hf.num_attention_heads)
        block_bytes = 2 * hf.num_hidden_layers * self.block_size * hf.num_key_value_heads * head_dim * hf.dtype.itemsize
        fit = int(total * cfg.gpu_memory_utilization - (total - free) - peak + current) // block_bytes
        if fit <= 0:
            raise RuntimeError("no memory left for the KV cache")
        cfg.kv_cache_num_blocks = min(fit, cfg.kv_cache_num_blocks)
        self.kv_cache = torch.empty(2, hf.num_hidden_layers, cfg.kv_cache_num_blocks, self.block_size,
                                    hf.num_key_value_heads, head_dim, dtype=hf.dtype, device=self.device)
        log.info("allocated %d KV blocks", cfg.kv_cache_num_blocks)
        layer = 0
        for module in self.model.modules():
            if hasattr(module, "k_cache") and hasattr(module, "v_cache"):
                module.k_cache, module.v_cache = self.kv_cache[0, layer], self.kv_cache[1, layer]
                layer += 1

    # ---- packing ---------------------------------------------------------------------------------
    @staticmethod
    def _per_seq(requests: list[Request]):
        b = len(requests)
        seq_len = np.fromiter((len(r.tokens) for r in requests), np.int32, b)
        nblk = np.fromiter((len(r.blocks) for r in requests), np.int32, b)
        blk_off = np.zeros(b + 1, np.int32)
        np.cumsum(nblk, out=blk_off[1:])
        blocks = np.fromiter(itertools.chain.from_iterable(r.blocks for r in requests), np.int32, int(blk_off[-1]))
        return seq_len, nblk, blk_off, blocks

    def _build_prefill_input(self, requests: list[Request]) -> tuple[torch.Tensor, Context]:
        b = len(requests)
        seq_len, nblk, blk_off, blocks = self._per_seq(requests)
        cached = np.fromiter((r.num_cached_tokens for r in requests), np.int32, b)
        q_len = seq_len - cached
        t = int(q_len.sum())
        new_tokens = np.fromiter(
            itertools.chain.from_iterable(r.tokens[r.num_cached_tokens:] if r.num_cached_tokens else r.tokens
                                          for r in requests), np.int32, t)
        items = self._prefill_items(q_len, seq_len)
        meta = self._stage.upload([seq_len, cached, blk_off, blocks, new_tokens, items.reshape(-1)])
        self.h2d_bytes += meta.numel() * 4
        width = max(int(nblk.max()), 1)
        out = ops.pack_prefill(meta, b, t, int(blk_off[-1]), width, self.block_size, bool(cached.any()), self.status)
        ctx = Context(prefill=True, positions=out["positions"], cu_seqlens_q=out["cu_seqlens_q"],
                      cu_seqlens_k=out["cu_seqlens_k"], slot_mapping=out["slot_mapping"],
                      max_seqlen_q=int(q_len.max()), max_seqlen_k=int(seq_len.max()),
                      block_table=out["block_table"], status=self.status,
                      prefill_items=meta[meta.numel() - items.size:].view(-1, 2) if items.size else None,
                      prefill_item_rows=self.item_rows)
        return out["input_ids"], ctx

    def _prefill_items(self, q_len: np.ndarray, seq_len: np.ndarray) -> np.ndarray:
        """The prefill kernel's work list for this step (ops.build_prefill_items): the host has the lengths in
        hand here, so the launch gets exactly its real (sequence, query block) items, longest first."""
        if not self.item_rows:
            return np.zeros((0, 2), np.int32)
        return ops.build_prefill_items(q_len, seq_len, self.item_rows)

    def _build_mixed_input(self, requests: list[Request], num_decode: int, slots: np.ndarray | None = None):
        """One ragged step: the first requests prefill, the last ``num_decode`` decode.  A decoding request
        is packed as a sequence whose first ``len - 1`` tokens are cached, so the prefill packing kernel
        lays out everything (ids, positions, slots, cu_seqlens, block table) for both parts at once."""
        b, bp = len(requests), len(requests) - num_decode
        seq_len, nblk, blk_off, blocks = self._per_seq(requests)
        cached = np.fromiter((r.num_cached_tokens for r in requests), np.int32, b)
        cached[bp:] = seq_len[bp:] - 1
        q_len = seq_len - cached
        t = int(q_len.sum())
        new_tokens = np.fromiter(
            itertools.chain(itertools.chain.from_iterable(r.tokens[r.num_cached_tokens:] for r in requests[:bp]),
                            (r.tokens[-1] for r in requests[bp:])), np.int32, t)
        items = self._prefill_items(q_len[:bp], seq_len[:bp])           # the prompts' part of the step
        meta = self._stage.upload([seq_len, cached, blk_off, blocks, new_tokens, items.reshape(-1)]
                                  + ([slots] if slots is not None else []))
        self.h2d_bytes += meta.numel() * 4
        width = max(int(nblk.max()), 1)
        out = ops.pack_prefill(meta, b, t, int(blk_off[-1]), width, self.block_size, True, self.status)
        cu_k = out["cu_seqlens_k"]
        items_end = meta.numel() - (b if slots is not None else 0)
        ctx = Context(prefill=True, positions=out["positions"], cu_seqlens_q=out["cu_seqlens_q"], cu_seqlens_k=cu_k,
                      slot_mapping=out["slot_mapping"], max_seqlen_q=int(q_len[:bp].max()),
                      max_seqlen_k=int(seq_len.max()), block_table=out["block_table"], num_decode=num_decode,
                      cache_seqlens=(cu_k[bp + 1:] - cu_k[bp:-1]).contiguous(), status=self.status,
                      prefill_items=meta[items_end - items.size:items_end].view(-1, 2) if items.size else None,
                      prefill_item_rows=self.item_rows)
        if slots is None:
            return out["input_ids"], ctx
        return out["input_ids"], ctx, meta[meta.numel() - b:]

    def _decode_meta(self, requests: list[Request]):
        b = len(requests)
        seq_len, nblk, blk_off, blocks = self._per_seq(requests)
        last = np.fromiter((r.tokens[-1] for r in requests), np.int32, b)
        meta = self._stage.upload([seq_len, blk_off, blocks, last, np.full(b, -1, np.int32)])
        self.h2d_bytes += meta.numel() * 4
        return meta, int(blk_off[-1]), int(nblk.max())

    def _build_decode_input(self, requests: list[Request]) -> tuple[torch.Tensor, Context]:
        b = len(requests)
        meta, nblocks, width = self._decode_meta(requests)
        gr = self.graph_runner
        if gr is not None and gr.max_batch_size >= b:
            padded = gr.padded_size(b)
            ops.pack_decode(meta, b, nblocks, width, self.block_size, gr.input_ids, gr.positions, gr.slot_mapping,
                            gr.cache_seqlens, gr.block_table, padded_seqs=padded, status=self.status)
            return gr.input_ids[:b], gr.static_context(b)
        dev = self.device
        ids, pos = torch.empty(b, dtype=torch.int64, device=dev), torch.empty(b, dtype=torch.int64, device=dev)
        slot, lens = torch.empty(b, dtype=torch.int32, device=dev), torch.empty(b, dtype=torch.int32, device=dev)
        table = torch.empty(b, width, dtype=torch.int32, device=dev)
        ops.pack_decode(meta, b, nblocks, width, self.block_size, ids, pos, slot, lens, table, status=self.status)
        return ids, Context(prefill=False, positions=pos, slot_mapping=slot, cache_seqlens=lens, block_table=table,
                            status=self.status)

    def _build_block_table(self, requests: list[Request]) -> torch.Tensor:
        """Block table alone, right-padded with -1 (executor.py:156-163); packed on the device."""
        b = len(requests)
        _, nblk, blk_off, blocks = self._per_seq(requests)
        zeros = np.zeros(b, np.int32)
        meta = self._stage.upload([zeros, zeros, blk_off, blocks])
        width = max(int(nblk.max()), 1)
        return ops.pack_prefill(meta, b, 0, int(blk_off[-1]), width, self.block_size, True, self.status)["block_table"]

    # ---- sampling -------------------------------------------------------------------------------
    def _build_sample_input(self, requests: list[Request]):
        """Tensors only when some request needs them (executor.py:165-191)."""
        temps = [r.sampling_params.temperature for r in requests]
        ks = [r.sampling_params.top_k for r in requests]
        ps = [r.sampling_params.top_p for r in requests]
        t = k = p = None
        if any(x > 0 for x in ks) or any(x < 1.0 for x in ps):
            k = torch.tensor(ks, dtype=torch.int32).pin_memory().to(self.device, non_blocking=True)
            p = torch.tensor(ps, dtype=torch.float32).pin_memory().to(self.device, non_blocking=True)
        if any(x != 1.0 for x in temps):
            t = torch.tensor(temps, dtype=torch.float32).pin_memory().to(self.device, non_blocking=True)
        return t, k, p

    def sample(self, logits: torch.Tensor, batch: Batch) -> list[int]:
        temperatures, top_k, top_p = self._build_sample_input(batch.requests)
        tokens = self.sampler(logits, temperatures, top_p=top_p, top_k=top_k)
        self.d2h_bytes += tokens.numel() * 8
        return tokens.tolist()

    def _tokens(self, hidden_rows: torch.Tensor, requests: list[Request], scatter_table=None, scatter_index=None):
        """The head of a step: token ids from the rows the lm_head reads.  A batch that only samples greedily (the
        reference's argmax path, sampler.py:31; a temperature does not move an argmax) takes the fused lm_head +
        argmax kernel; otherwise lm_head, then the sampler."""
        temperatures, top_k, top_p = self._build_sample_input(requests)
        rows = hidden_rows.shape[0]
        if self.fused_head and top_k is None and top_p is None and rows <= self.fused_head_max_rows:
            return self.model.greedy_tokens(hidden_rows, self._head_scratch, scatter_table=scatter_table,
                                            scatter_index=scatter_index, status=self.status)
        logits = self.model.lm_head(hidden_rows)
        return self.sampler(logits, temperatures, top_p=top_p, top_k=top_k, scatter_table=scatter_table,
                            scatter_index=scatter_index)

    # ---- pipelined step: nothing comes back to the host ---------------------------------------------
    def ensure_token_table(self, num_slots: int) -> None:
        if self.token_table.numel() < num_slots:
            grown = torch.zeros(max(num_slots, 2 * self.token_table.numel()), dtype=torch.int64, device=self.device)
            grown[:self.token_table.numel()] = self.token_table
            self.token_table = grown

    @torch.inference_mode()
    def launch(self, batch: Batch, slots: np.ndarray):
        """Enqueue one step.  The sampled tokens go to ``token_table[slots]`` on the device (the next
        decode packing reads its input ids from there) and, asynchronously, to a pinned host buffer.

        Returns ``(pinned int64 view, event)``: the view holds the tokens once the event has completed.
        Decode input tokens are NOT taken from ``Request.tokens`` (they may still be placeholders).
        """
        reqs, b = batch.requests, len(batch.requests)
        self._step += 1
        if batch.type == Batch.PREFILL:
            seq_len, nblk, blk_off, blocks = self._per_seq(reqs)
            cached = np.fromiter((r.num_cached_tokens for r in reqs), np.int32, b)
            q_len = seq_len - cached
            t = int(q_len.sum())
            new_tokens = np.fromiter(
                itertools.chain.from_iterable(r.tokens[r.num_cached_tokens:] if r.num_cached_tokens else r.tokens
                                              for r in reqs), np.int32, t)
            meta = self._stage.upload([seq_len, cached, blk_off, blocks, new_tokens, slots])
            slots_dev = meta[meta.numel() - b:]
            width = max(int(nblk.max()), 1)
            out = ops.pack_prefill(meta, b, t, int(blk_off[-1]), width, self.block_size, bool(cached.any()), self.status)
            ctx = Context(prefill=True, positions=out["positions"], cu_seqlens_q=out["cu_seqlens_q"],
                          cu_seqlens_k=out["cu_seqlens_k"], slot_mapping=out["slot_mapping"],
                          max_seqlen_q=int(q_len.max()), max_seqlen_k=int(seq_len.max()),
                          block_table=out["block_table"], status=self.status)
            input_ids = out["input_ids"]
        elif batch.type == Batch.MIXED:                # (its decode inputs come from Request.tokens: the caller has
            input_ids, ctx, slots_dev = self._build_mixed_input(reqs, batch.num_decode, slots)   # resolved them)
            meta = None
        else:
            seq_len, nblk, blk_off, blocks = self._per_seq(reqs)
            meta = self._stage.upload([seq_len, blk_off, blocks, np.zeros(b, np.int32), slots])
            slots_dev = meta[meta.numel() - b:]
            nblocks, width = int(blk_off[-1]), int(nblk.max())
            gr = self.graph_runner
            if gr is not None and gr.max_batch_size >= b:
                ops.pack_decode(meta, b, nblocks, width, self.block_size, gr.input_ids, gr.positions, gr.slot_mapping,
                                gr.cache_seqlens, gr.block_table, padded_seqs=gr.padded_size(b),
                                prev_sampled=self.token_table, status=self.status)
                input_ids, ctx = gr.input_ids[:b], gr.static_context(b)
            else:
                dev = self.device
                input_ids, pos = torch.empty(b, dtype=torch.int64, device=dev), torch.empty(b, dtype=torch.int64, device=dev)
                slot, lens = torch.empty(b, dtype=torch.int32, device=dev), torch.empty(b, dtype=torch.int32, device=dev)
                table = torch.empty(b, width, dtype=torch.int32, device=dev)
                ops.pack_decode(meta, b, nblocks, width, self.block_size, input_ids, pos, slot, lens, table,
                                prev_sampled=self.token_table, status=self.status)
                ctx = Context(prefill=False, positions=pos, slot_mapping=slot, cache_seqlens=lens, block_table=table,
                              status=self.status)
        if meta is not None:
            self.h2d_bytes += meta.numel() * 4
        tokens = self._tokens(self.forward(ctx, input_ids, head=False), reqs, self.token_table, slots_dev)
        host = self._out_ring[self._step % self.RING, :b]
        host.copy_(tokens, non_blocking=True)
        self.d2h_bytes += b * 8
        event = torch.cuda.Event()
        event.record()
        return host, event

    # ---- forward ---------------------------------------------------------------------------------
    def prefill(self, ctx: Context, input_ids: torch.Tensor, head: bool = True) -> torch.Tensor:
        return self.model(ctx, input_ids, ctx.positions, head=head)

    def decode(self, ctx: Context, input_ids: torch.Tensor, head: bool = True) -> torch.Tensor:
        gr = self.graph_runner
        if gr is not None and gr.max_batch_size >= input_ids.size(0):
            rows = gr.replay(ctx, input_ids)                   # the captured step ends in front of the head
            return self.model.lm_head(rows) if head else rows
        return self.model(ctx, input_ids, ctx.positions, head=head)

    def forward(self, ctx: Context, tokens: torch.Tensor, head: bool = True) -> torch.Tensor:
        """Logits (``head=True``, the reference's contract, executor.py:197-214) or the rows the head reads."""
        return self.prefill(ctx, tokens, head) if ctx.prefill else self.decode(ctx, tokens, head)

    @torch.inference_mode()
    def execute(self, batch: Batch) -> list[int]:
        self._step += 1
        if batch.type == Batch.PREFILL:
            input_ids, ctx = self._build_prefill_input(batch.requests)
        elif batch.type == Batch.MIXED:
            input_ids, ctx = self._build_mixed_input(batch.requests, batch.num_decode)
        else:
            input_ids, ctx = self._build_decode_input(batch.requests)
        tokens = self._tokens(self.forward(ctx, input_ids, head=False), batch.requests)
        self.d2h_bytes += tokens.numel() * 8
        return tokens.tolist()

    def check_device_status(self) -> None:
        """Synchronising check of the kernels' error word (bad slots / block ids / positions)."""
        ops.check_status(self.status)
