"""Engine: the user-facing loop (``submit`` / ``step`` / ``generate``), as in
``minivllm/engine/engine.py:14-90``.  Prompts are token-id lists.  A tokenizer is optional: with
a checkpoint directory the completions are decoded to text like the reference does; for
random-init shape configs (no tokenizer on disk) ``prompt``/``completion`` are left ``None``.
"""
from __future__ import annotations

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

    def generate(self, prompts: list[list[int]], sampling_params, use_tqdm: bool = True) -> list[dict]:
        if not isinstance(sampling_params, list):
            sampling_params = [sampling_params] * len(prompts)
        for prompt, sp in zip(prompts, sampling_params):
            self.submit(prompt, sp)
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
        done.sort(key=lambda r: r.id)
        dec = self.tokenizer.decode if self.tokenizer is not None else (lambda toks: None)
        return [{"prompt": dec(r.prompt_tokens), "completion": dec(r.completion_tokens),
                 "tokens": r.completion_tokens} for r in done]
