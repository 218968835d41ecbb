"""A scheduled step: all-prefill or all-decode (minivllm/scheduler/batch.py:4-12); with
``Config.enable_mixed_steps`` also MIXED: ``requests`` = the prompts to prefill followed by the last
``num_decode`` requests, which decode."""
import time


class Batch:
    PREFILL, DECODE, MIXED = 0, 1, 2

    def __init__(self, typ: int, reqs: list, num_decode: int = 0):
        self.type = typ
        self.requests = reqs
        self.num_decode = num_decode if typ == Batch.MIXED else (len(reqs) if typ == Batch.DECODE else 0)
        self.create_time = time.perf_counter()
