"""One generation request (same observable fields as minivllm/engine/request.py:7-47)."""
from __future__ import annotations

import itertools
from typing import List, Optional

from ..config.sampling import SamplingParams

_ids = itertools.count()


class Request:
    WAITING, RUNNING, FINISHED = 0, 1, 2

    def __init__(self, prompt_tokens: List[int], sampling_params: Optional[SamplingParams] = None):
        self.id = next(_ids)
        self.state = Request.WAITING
        self.tokens = list(prompt_tokens)
        self.prompt_token_count = len(self.tokens)
        self.sampling_params = sampling_params if sampling_params is not None else SamplingParams()
        self.blocks: List[int] = []          # ids of the KV blocks holding this request's keys/values
        self.num_cached_tokens = 0           # leading tokens found in the prefix cache (skip prefill)

    def __len__(self) -> int:
        return len(self.tokens)

    def __getitem__(self, i):
        return self.tokens[i]

    def append_output_token(self, token: int) -> None:
        self.tokens.append(token)

    @property
    def finished(self) -> bool:
        return self.state == Request.FINISHED

    @property
    def prompt_tokens(self) -> List[int]:
        return self.tokens[:self.prompt_token_count]

    @property
    def completion_tokens(self) -> List[int]:
        return self.tokens[self.prompt_token_count:]

    @property
    def num_completion_tokens(self) -> int:
        return len(self.tokens) - self.prompt_token_count
