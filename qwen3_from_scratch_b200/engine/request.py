"""A generation request and its sampling parameters.

Reference: inference/sequence.py:12-49 (prompt, generated tokens, progress pointer, status),
factory/batch_config.py:83-91 (temperature, top_k, max_new_tokens).
"""

from __future__ import annotations

import enum
import itertools
from dataclasses import dataclass, field
from typing import List, Optional

_ids = itertools.count()


class RequestStatus(enum.Enum):
    WAITING = 0
    RUNNING = 1
    FINISHED = 2


@dataclass
class SamplingParams:
    """temperature <= 0: greedy.  top_k > 0 with a temperature: draw among the k largest.
    seed: with the request's key and the position it fixes every draw."""

    temperature: float = 0.0
    top_k: int = 0
    max_new_tokens: int = 100
    ignore_eos: bool = False
    seed: int = 0


@dataclass
class Request:
    prompt: List[int]
    params: SamplingParams = field(default_factory=SamplingParams)
    request_id: Optional[str] = None
    key: Optional[int] = None  # keys the random stream; defaults to the running number of the request

    def __post_init__(self):
        n = next(_ids)
        if self.request_id is None:
            self.request_id = f"req-{n}"
        if self.key is None:
            self.key = n
        self.prompt = [int(t) for t in self.prompt]
        if not self.prompt:
            raise ValueError("a request needs at least one prompt token")
        self.output: List[int] = []
        self.num_computed = 0  # tokens of prompt + output whose keys/values are in the cache
        self.num_scheduled = 0  # tokens the scheduler gave it in the current step
        self.status = RequestStatus.WAITING
        self.finish_reason: Optional[str] = None  # "eos" | "length"
        self.preemptions = 0
        self.arrival_time: Optional[float] = None
        self.first_token_time: Optional[float] = None
        self.finish_time: Optional[float] = None

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    def __len__(self) -> int:
        return len(self.prompt) + len(self.output)

    @property
    def remaining(self) -> int:
        """Tokens not yet in the cache; 1 in steady decoding."""
        return len(self) - self.num_computed

    @property
    def is_decoding(self) -> bool:
        return self.remaining == 1 and self.num_computed > 0

    def next_tokens(self, n: int) -> List[int]:
        start, plen = self.num_computed, len(self.prompt)
        if start + n <= plen:
            return self.prompt[start:start + n]
        if start >= plen:
            return self.output[start - plen:start - plen + n]
        return self.prompt[start:] + self.output[:start + n - plen]

    def __hash__(self):
        return hash(self.request_id)

    def __eq__(self, other):
        return isinstance(other, Request) and other.request_id == self.request_id
