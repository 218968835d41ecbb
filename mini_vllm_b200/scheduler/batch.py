"""A scheduled step: all-prefill or all-decode (minivllm/scheduler/batch.py:4-12)."""
import time


class Batch:
    PREFILL, DECODE = 0, 1

    def __init__(self, typ: int, reqs: list):
        self.type = typ
        self.requests = reqs
        self.create_time = time.perf_counter()
