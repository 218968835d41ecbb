"""Engine: the user-facing loop (``submit`` / ``step`` / ``generate``), as in
``minivllm/engine/engine.py:14-90``.  Prompts are token-id lists.  A tokenizer is optional: with
a checkpoint directory the completions are decoded to text like the reference does; for
random-init shape configs (no tokenizer on disk) ``prompt``/``completion`` are left ``None``.
"""
from __future__ import annotations

from collections import deque

import numpy as np
import torch

from ..config.config import Config
from ..config.sampling import SamplingParams
from ..executor.executor import Executor
from ..scheduler.batch import Batch
from ..scheduler.scheduler import Scheduler
from .metrics import Metrics
from .request import Request


class Engine:
    def __init__(self, config: Config):
        self.config = config
        self.tokenizer = None
        if config.model is not None:
            from transformers import AutoTokenizer
            self.tokenizer = AutoTokenizer.from_pretrained(config.model, use_fast=True)
        self.executor = Executor(config)       # may lower config.kv_cache_num_blocks to what fits
        self.scheduler = Scheduler(config)
        self.metrics = Metrics()

    def submit(self, tokens: list[int], sampling_params: SamplingParams) -> Request:
        req = Request(tokens, sampling_params)
        self.scheduler.submit(req)
        return req

    def step(self) -> Batch:
        batch = self.scheduler.schedule()
        if batch is None:
            raise RuntimeError("nothing can be scheduled: a request needs more KV blocks than the pool holds")
        tokens = self.executor.execute(batch)
        self.scheduler.update(batch, tokens)
        self.metrics.update(batch)
        return batch

    @property
    def finished(self) -> bool:
        return self.scheduler.finished

    PLACEHOLDER = -1      # stands in Request.tokens for a sampled id that has not reached the host yet
    RUN_AHEAD = 2         # steps the host may be ahead of the device results

    def _schedule_is_token_independent(self, sampling_params) -> bool:
        """True when the step loop may run ahead of the sampled tokens - always, by now: a request that has
        emitted EOS is found out a few steps late and what it generated past that point is dropped; a block
        is published to the prefix cache when its last tokens have reached the host; a mixed step takes its
        decode inputs from ``Request.tokens``, so the loop catches up with the device before one."""
        return True

    def _generate_pipelined(self, reqs: list[Request]) -> None:
        """The step loop without the per-step device-to-host sync (the reference blocks on ``.tolist()``
        every step, executor.py:193-195).  Sampled ids stay on the device, where the next decode packing
        picks them up; they reach ``Request.tokens`` a few steps late through a pinned buffer.

        Requests that stop on EOS are scheduled speculatively: until the EOS token has reached the host
        (at most ``RUN_AHEAD`` steps) the request keeps decoding; then it is cut back to the EOS token and
        its blocks are freed.  Freeing while those extra steps may still be in flight is safe because every
        step runs on one stream: whoever gets the blocks next writes them after the stragglers have."""
        ex, sch = self.executor, self.scheduler
        eos = self.config.eos_token_ids or ()
        prefix_cache, block_size = bool(self.config.enable_prefix_cache), self.config.kv_cache_block_size
        slot_of = {r.id: i for i, r in enumerate(reqs)}
        ex.ensure_token_table(len(reqs))
        unresolved = dict.fromkeys(slot_of, 0)
        stopped_at: dict[int, int] = {}               # request id -> number of tokens it really has (EOS included)
        pending: deque = deque()

        def resolve(item) -> None:
            batch_reqs, positions, host, event = item
            event.synchronize()
            for r, pos, tok in zip(batch_reqs, positions, host.tolist()):
                unresolved[r.id] -= 1
                if r.id in stopped_at:                # a step that ran past the request's EOS
                    continue
                r.tokens[pos] = tok
                if prefix_cache and (pos + 1) % block_size == 0:
                    sch.block_manager.cache_block_at(r, (pos + 1) // block_size - 1)
                if eos and tok in eos and not r.sampling_params.ignore_eos:
                    stopped_at[r.id] = pos + 1
                    del r.tokens[pos + 1:]
                    if not r.finished:
                        sch.stop(r)

        timed = torch.cuda.is_available()             # (the loop itself is host logic and also runs without a GPU)
        if timed:
            self._job_start = torch.cuda.Event(enable_timing=True)
            self._job_start.record()
        while not self.finished:
            if prefix_cache and pending:
                # A preempted request waits at the head of the queue with its last sampled ids possibly still
                # placeholders.  Admission hashes a prompt's full blocks into the prefix cache, so those ids
                # must be real before the scheduler sees the request again.
                for r in sch.waiting:
                    if r.num_completion_tokens == 0:  # never started: everything behind it is fresh too
                        break
                    if unresolved[r.id]:
                        while pending:
                            resolve(pending.popleft())
                        break
            batch = sch.schedule()
            if batch is None:
                raise RuntimeError("nothing can be scheduled: a request needs more KV blocks than the pool holds")
            if batch.type != Batch.DECODE and any(unresolved[r.id] for r in batch.requests):
                while pending:                      # a preempted request is re-prefilled from its real tokens
                    resolve(pending.popleft())
                if any(r.finished for r in batch.requests):   # ... unless those tokens ended in an EOS
                    bp = len(batch.requests) - (batch.num_decode if batch.type == Batch.MIXED else 0)
                    head = [r for r in batch.requests[:bp] if not r.finished]
                    tail = [r for r in batch.requests[bp:] if not r.finished]
                    if not head and not tail:
                        continue
                    batch.requests, batch.num_decode = head + tail, len(tail)
                    if batch.type == Batch.MIXED and not (head and tail):
                        batch.type = Batch.PREFILL if head else Batch.DECODE
            slots = np.fromiter((slot_of[r.id] for r in batch.requests), np.int32, len(batch.requests))
            host, event = ex.launch(batch, slots)
            positions = [len(r.tokens) for r in batch.requests]
            for r in batch.requests:
                unresolved[r.id] += 1
            sch.update(batch, [self.PLACEHOLDER] * len(batch.requests), defer_cache=True)
            self.metrics.update(batch)
            pending.append((list(batch.requests), positions, host, event))
            while len(pending) > self.RUN_AHEAD:
                resolve(pending.popleft())
        if timed:
            self._job_end = torch.cuda.Event(enable_timing=True)
            self._job_end.record()
        while pending:
            resolve(pending.popleft())

    @property
    def last_job_device_ms(self) -> float:
        """Device time between the first and the last kernel of the last pipelined ``generate``."""
        self._job_end.synchronize()
        return self._job_start.elapsed_time(self._job_end)

    def generate(self, prompts: list[list[int]], sampling_params, use_tqdm: bool = True) -> list[dict]:
        if not isinstance(sampling_params, list):
            sampling_params = [sampling_params] * len(prompts)
        reqs = [self.submit(prompt, sp) for prompt, sp in zip(prompts, sampling_params)]
        if not use_tqdm and self._schedule_is_token_independent(sampling_params):
            self._generate_pipelined(reqs)
            self.executor.check_device_status()    # every result is on the host by now: the read costs no extra sync
            dec = self.tokenizer.decode if self.tokenizer is not None else (lambda toks: None)
            return [{"prompt": dec(r.prompt_tokens), "completion": dec(r.completion_tokens),
                     "tokens": r.completion_tokens} for r in sorted(reqs, key=lambda r: r.id)]
        pbar = None
        if use_tqdm:
            from tqdm.auto import tqdm
            pbar = tqdm(total=len(prompts), desc="Generating", dynamic_ncols=True)
        done: list[Request] = []
        shown = 0
        while not self.finished:
            batch = self.step()
            done.extend(r for r in batch.requests if r.finished)
            if pbar is not None:
                s = self.metrics.stats()
                pbar.set_postfix({"Prefill(token/s)": f"{s.prefill_throughput:4.0f}",
                                  "Decode(token/s)": f"{s.decode_throughput:4.0f}",
                                  "TTFT": f"{s.time_to_first_token:4.2f}", "ITL": f"{s.inter_token_latency:4.2f}"})
                pbar.update(len(done) - shown)
                shown = len(done)
        if pbar is not None:
            pbar.close()
        self.executor.check_device_status()        # a kernel that skipped a bad access or gave up a wait says so here
        done.sort(key=lambda r: r.id)
        dec = self.tokenizer.decode if self.tokenizer is not None else (lambda toks: None)
        return [{"prompt": dec(r.prompt_tokens), "completion": dec(r.completion_tokens),
                 "tokens": r.completion_tokens} for r in done]


LLM = Engine      # the name offline-inference scripts use for this class
