"""Throughput bookkeeping with the meanings of minivllm/engine/metrics.py:27-70: step time is
schedule-to-update wall time; TTFT is the mean prefill step, ITL the mean decode step."""
from __future__ import annotations

import time
from dataclasses import dataclass

from ..scheduler.batch import Batch


@dataclass
class Stats:
    prefill_throughput: float = 0.0
    decode_throughput: float = 0.0
    time_to_first_token: float = 0.0
    inter_token_latency: float = 0.0
    tokens_per_second: float = 0.0
    requests_per_second: float = 0.0
    finished_requests: int = 0


class Metrics:
    def __init__(self):
        self.reset()
        self.prefill_tokens = self.decode_tokens = 0

    def reset(self) -> None:
        self.prefill_time = self.decode_time = 0.0
        self.prefill_steps = self.decode_steps = 0
        self.finished_request_count = 0
        self.start_time = time.perf_counter()

    def update(self, batch: Batch) -> None:
        dt = time.perf_counter() - batch.create_time
        if batch.type == Batch.MIXED:                 # counted as a decode step that also prefilled
            bp = len(batch.requests) - batch.num_decode
            self.prefill_tokens += sum(len(r.tokens) - 1 - r.num_cached_tokens for r in batch.requests[:bp])
            self.decode_steps += 1
            self.decode_time += dt
            self.decode_tokens += batch.num_decode
            self.finished_request_count += sum(1 for r in batch.requests if r.finished)
        elif batch.type == Batch.PREFILL:
            self.prefill_steps += 1
            self.prefill_time += dt
            self.prefill_tokens += sum(len(r.tokens) - r.num_cached_tokens for r in batch.requests)
        else:
            self.decode_steps += 1
            self.decode_time += dt
            self.decode_tokens += len(batch.requests)
            self.finished_request_count += sum(1 for r in batch.requests if r.finished)

    def stats(self) -> Stats:
        elapsed = time.perf_counter() - self.start_time
        div = lambda a, b: a / b if b > 0 else 0.0
        return Stats(prefill_throughput=div(self.prefill_tokens, self.prefill_time),
                     decode_throughput=div(self.decode_tokens, self.decode_time),
                     time_to_first_token=div(self.prefill_time, self.prefill_steps),
                     inter_token_latency=div(self.decode_time, self.decode_steps),
                     tokens_per_second=div(self.prefill_tokens + self.decode_tokens, elapsed),
                     requests_per_second=div(self.finished_request_count, elapsed),
                     finished_requests=self.finished_request_count)
