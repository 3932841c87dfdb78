"""Requests: sampling options, the life cycle, token bookkeeping and stop rules.

The states, the legal transitions and the stop rules are the reference's
(src/infurnace/engine/request.py:7-33,95-103,123-134); one transition is added, from a
running state back to WAITING, which is what preemption does when pages run out.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from time import monotonic
from typing import List, Optional


class RequestState(Enum):
    WAITING = "waiting"
    PREFILLING = "prefilling"
    DECODING = "decoding"
    FINISHED = "finished"
    CANCELLED = "cancelled"
    FAILED = "failed"
    REJECTED = "rejected"


TERMINAL = frozenset({RequestState.FINISHED, RequestState.CANCELLED, RequestState.FAILED, RequestState.REJECTED})

_NEXT = {
    RequestState.WAITING: {RequestState.PREFILLING, RequestState.CANCELLED, RequestState.FAILED, RequestState.REJECTED},
    RequestState.PREFILLING: {RequestState.DECODING, RequestState.FINISHED, RequestState.CANCELLED,
                              RequestState.FAILED, RequestState.WAITING},
    RequestState.DECODING: {RequestState.FINISHED, RequestState.CANCELLED, RequestState.FAILED, RequestState.WAITING},
    RequestState.FINISHED: set(), RequestState.CANCELLED: set(), RequestState.FAILED: set(), RequestState.REJECTED: set(),
}


@dataclass
class SamplingParams:
    """The reference's fields (request.py:35-44) plus ``seed``.

    ``temperature`` 0 is greedy (the reference's only sampler, src/infurnace/sampler/greedy.py:21-22);
    above 0 a token is drawn from softmax(logits / temperature).  ``top_k`` and ``top_p``
    exist in the reference but nothing there reads them; here ``top_k`` may be 0 (off) or 1
    (greedy whatever the temperature) and ``top_p`` must be 1.0; other values are refused
    at admission."""
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    max_tokens: int = 128
    stop_token_ids: List[int] = field(default_factory=list)
    min_tokens: int = 0
    include_stop_str_in_output: bool = False
    seed: int = 0

    def problem(self) -> Optional[str]:
        if not self.temperature >= 0.0:
            return f"temperature {self.temperature} is negative"
        if self.top_k not in (0, 1):
            return f"top_k {self.top_k} is not supported (0: off, 1: greedy)"
        if self.top_p != 1.0:
            return f"top_p {self.top_p} is not supported (1.0: off)"
        if self.max_tokens < 0:
            return f"max_tokens {self.max_tokens} is negative"
        return None

    @property
    def effective_temperature(self) -> float:
        return 0.0 if self.top_k == 1 else float(self.temperature)


@dataclass
class RequestMetrics:
    arrival_time: float = field(default_factory=monotonic)
    first_token_time: Optional[float] = None
    completion_time: Optional[float] = None

    @property
    def ttft(self) -> Optional[float]:
        return None if self.first_token_time is None else self.first_token_time - self.arrival_time

    @property
    def total_latency(self) -> Optional[float]:
        return None if self.completion_time is None else self.completion_time - self.arrival_time


@dataclass
class Request:
    request_id: str
    prompt_token_ids: List[int]
    sampling_params: SamplingParams = field(default_factory=SamplingParams)
    context_limit: Optional[int] = None
    eos_token_ids: List[int] = field(default_factory=list)
    prompt: Optional[str] = None
    stop_strings: List[str] = field(default_factory=list)

    state: RequestState = RequestState.WAITING
    error: Optional[str] = None
    finish_reason: Optional[str] = None
    metrics: RequestMetrics = field(default_factory=RequestMetrics)
    num_computed_tokens: int = 0          # tokens whose keys and values are in pages
    num_preemptions: int = 0
    admission_index: int = -1

    def __post_init__(self):
        self.prompt_token_ids = [int(t) for t in self.prompt_token_ids]
        self._output: List[int] = []
        self._all: List[int] = list(self.prompt_token_ids)

    @property
    def output_token_ids(self):
        return tuple(self._output)

    @property
    def all_token_ids(self):
        return tuple(self._all)

    @property
    def num_tokens(self) -> int:
        return len(self._all)

    def transition(self, new: RequestState) -> None:
        if new not in _NEXT[self.state]:
            raise ValueError(f"invalid transition: {self.state} -> {new}")
        if new in TERMINAL:
            self.metrics.completion_time = monotonic()
        self.state = new

    def is_terminal(self) -> bool:
        return self.state in TERMINAL

    def is_active(self) -> bool:
        return self.state in (RequestState.PREFILLING, RequestState.DECODING)

    def append_output_token(self, token_id: int) -> None:
        if self.metrics.first_token_time is None:
            self.metrics.first_token_time = monotonic()
        self._output.append(int(token_id))
        self._all.append(int(token_id))

    def check_finished(self, new_token_id: int) -> Optional[str]:
        """The stop reason after ``new_token_id`` or None, in the reference's order
        (request.py:123-134): the min_tokens floor first, then eos, stop ids, max_tokens."""
        sp = self.sampling_params
        if len(self._output) < sp.min_tokens:
            return None
        if new_token_id in self.eos_token_ids:
            return "eos"
        if new_token_id in sp.stop_token_ids:
            return "stop_token_ids"
        if len(self._output) >= sp.max_tokens:
            return "max_tokens"
        return None
