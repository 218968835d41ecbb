"""Continuous-batching scheduler: prefill-first, FCFS, newest-first preemption.

Same decisions, in the same order, as ``minivllm/scheduler/scheduler.py`` — the order of
``Batch.requests`` is the row order of every packed tensor:

* a step is all-prefill if any waiting request fits, otherwise all-decode (``:83-89``);
* prefill admits from the head of ``waiting`` while the sequence count, the token budget
  (uncached tokens, evaluated before allocation, i.e. the full length) and the free blocks allow
  (``:34-56``);
* decode visits ``running`` from the left; when a request needs a block that is not there the
  right-most running request is preempted (freed, pushed to the FRONT of ``waiting``), and the
  request itself if it is the only one left (``:59-81,91-98``);
* ``update`` appends the sampled token, finishes on ``max_tokens`` or EOS (unless ``ignore_eos``)
  and otherwise publishes a just-filled block to the prefix cache (``:101-112``).
"""
from __future__ import annotations

from collections import deque

from ..engine.request import Request
from ..kvcache.block_manager import KVCacheBlockManager
from .batch import Batch


class Scheduler:
    def __init__(self, config):
        self.max_num_batched_seqs = config.max_num_batched_seqs
        self.max_num_batched_tokens = config.max_num_batched_tokens
        self.eos_token_ids = config.eos_token_ids
        self.mixed_steps = bool(getattr(config, "enable_mixed_steps", False))
        prefix = bool(getattr(config, "enable_prefix_cache", False))
        self.block_manager = KVCacheBlockManager(config.kv_cache_num_blocks, config.kv_cache_block_size,
                                                 support_prefix_cache=prefix, keep_last_block_uncached=prefix)
        self.waiting: deque[Request] = deque()
        self.running: deque[Request] = deque()

    @property
    def finished(self) -> bool:
        return not (self.waiting or self.running)

    def submit(self, req: Request) -> None:
        self.waiting.append(req)

    def preempt(self, req: Request) -> None:
        req.state = Request.WAITING
        self.block_manager.deallocate(req)
        self.waiting.appendleft(req)

    def _schedule_prefill(self, max_seqs: int | None = None, max_tokens: int | None = None):
        bm, picked = self.block_manager, []
        budget = self.max_num_batched_tokens if max_tokens is None else max_tokens
        max_seqs = self.max_num_batched_seqs if max_seqs is None else max_seqs
        while self.waiting and len(picked) < max_seqs:
            req = self.waiting[0]
            cost = len(req.tokens) - req.num_cached_tokens
            if cost > budget or not bm.can_allocate_new_block(req):
                break
            budget -= cost
            bm.allocate_blocks_for_prefill(req)
            req.state = Request.RUNNING
            self.running.append(self.waiting.popleft())
            picked.append(req)
        return Batch(Batch.PREFILL, picked) if picked else None

    def _schedule_decode(self):
        bm, picked = self.block_manager, []
        while self.running and len(picked) < self.max_num_batched_seqs:
            req = self.running.popleft()
            while not bm.can_allocate_new_block(req):
                if not self.running:
                    self.preempt(req)
                    break
                self.preempt(self.running.pop())
            if req.state == Request.RUNNING:
                bm.allocate_block_for_decode(req)
                picked.append(req)
        if not picked:
            return None
        self.running.extendleft(reversed(picked))
        return Batch(Batch.DECODE, picked)

    def _schedule_mixed(self):
        """Extension (the reference's step is prefill XOR decode, ``:83-89``): the running requests
        decode as usual and, in the same step, prompts are admitted from the head of ``waiting`` with the
        sequence slots and the token budget the decodes leave."""
        decode = self._schedule_decode()
        nd = len(decode.requests) if decode else 0
        prefill = self._schedule_prefill(self.max_num_batched_seqs - nd, self.max_num_batched_tokens - nd)
        if prefill is None or decode is None:
            return prefill or decode
        return Batch(Batch.MIXED, prefill.requests + decode.requests, num_decode=nd)

    def schedule(self):
        if self.mixed_steps and self.running and self.waiting:
            return self._schedule_mixed()
        return self._schedule_prefill() or self._schedule_decode()

    def stop(self, req: Request) -> None:
        """Ends a request from outside a step (the pipelined loop learns of an EOS a few steps late)."""
        if req.state == Request.RUNNING:
            self.block_manager.deallocate(req)
            self.running.remove(req)
        elif req.state == Request.WAITING:            # preempted in the meantime: it holds no blocks
            self.waiting.remove(req)
        req.state = Request.FINISHED

    def update(self, batch: Batch, tokens: list[int], defer_cache: bool = False) -> None:
        """``defer_cache``: the tokens are placeholders (pipelined engine); blocks that fill up are published
        later, by ``block_manager.cache_block_at``, when their tokens are known."""
        bm = self.block_manager
        for req, token in zip(batch.requests, tokens):
            req.append_output_token(token)
            sp = req.sampling_params
            hit_eos = bool(self.eos_token_ids) and token in self.eos_token_ids and not sp.ignore_eos
            if req.num_completion_tokens >= sp.max_tokens or hit_eos:
                req.state = Request.FINISHED
                bm.deallocate(req)
                self.running.remove(req)
            elif not defer_cache:
                bm.cache_block_if_needed(req)
