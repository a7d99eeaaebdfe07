"""Requests and their life cycle (andre-fu/prism engine/request_manager.py:10-59:
``QUEUED -> PREFILLING -> DECODING -> DONE`` with ttft / tbt timing).  A
preempted request goes back to the front of the waiting queue and is
recomputed from its prompt plus what it has generated."""

from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import List, Optional

from ..sampling.sampler import SamplingParams


class RequestState(Enum):
    WAITING = "waiting"            # QUEUED in the reference
    PREFILLING = "prefilling"
    DECODING = "decoding"
    FINISHED = "finished"          # DONE in the reference


@dataclass
class Request:
    id: int
    prompt_tokens: List[int]
    params: SamplingParams
    state: RequestState = RequestState.WAITING
    generated_tokens: List[int] = field(default_factory=list)
    num_computed: int = 0                 # tokens of prompt + generated whose keys are in the cache
    finish_reason: Optional[str] = None   # "stop" | "length"
    error: Optional[str] = None
    num_preemptions: int = 0
    arrival_time: float = 0.0
    first_token_time: float = 0.0
    done_time: float = 0.0

    @property
    def tokens(self) -> List[int]:
        return self.prompt_tokens + self.generated_tokens

    def next_tokens(self, n: int) -> List[int]:
        """The ``n`` tokens after the ``num_computed`` ones already in the cache."""
        a, np_ = self.num_computed, len(self.prompt_tokens)
        if a >= np_:
            return self.generated_tokens[a - np_:a - np_ + n]
        if a + n <= np_:
            return self.prompt_tokens[a:a + n]
        return self.prompt_tokens[a:] + self.generated_tokens[:a + n - np_]

    @property
    def remaining(self) -> int:
        return len(self.prompt_tokens) + len(self.generated_tokens) - self.num_computed

    @property
    def ttft(self) -> float:
        """Time to first token, seconds (request_manager.py:40-44)."""
        return self.first_token_time - self.arrival_time if self.first_token_time > 0 else 0.0

    @property
    def tbt(self) -> float:
        """Mean time between tokens, seconds (request_manager.py:53-59)."""
        n = len(self.generated_tokens)
        if n <= 1 or self.first_token_time <= 0 or self.done_time <= 0:
            return 0.0
        return (self.done_time - self.first_token_time) / (n - 1)


@dataclass
class GenerationResult:
    token_ids: List[int]
    finish_reason: Optional[str]
    ttft: float
    tbt: float
    num_preemptions: int = 0
    error: Optional[str] = None
