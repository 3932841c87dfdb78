"""The scheduler: admission, portions of prompts under a token budget, decoding,
finishing, and what happens when pages run out.

The reference admits a request only if a whole slot is free, runs one request's prefill
at a time and decodes only when no prefill is pending (src/infurnace/scheduler/scheduler.py:
39-62,97-114); its documents ask for mixed steps under a token budget with decode first
(docs/roadmap.md:371-375).  This scheduler plans one step at a time:

1. every DECODING request gets its one token;
2. what is left of the token budget goes to PREFILLING requests, oldest first, each
   taking ``min(rest of its tokens, budget left, max_prefill_portion)``;
3. then to waiting requests, in arrival order, while a state slot and pages for at
   least their first tokens are free.

It works on numbers only: token counts, page counts, states.  Pages are counted through
the cache manager's accounting; the step function takes them when the step runs.

When pages run out.  If a DECODING request cannot get the page its next token needs, the
running request that was admitted last is preempted: its pages and state slot go back,
its progress is set to zero, it keeps the tokens it has generated and goes to the front
of the waiting queue; when it runs again it recomputes prompt and generated tokens.  The
victim is a function of admission order only.  A request that cannot advance although it
is the only one running has met a pool that is too small for it and FAILS with "out of KV
pages".  A PREFILLING request that finds too few pages takes the tokens that fit, or
waits a step.  Waiting requests wait.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional

from ..errors import SchedulerError
from .request import Request, RequestState


@dataclass(frozen=True)
class PlannedEntry:
    request_id: str
    start: int                  # position of the first token of the span
    tokens: tuple               # the span
    sample: bool                # the span reaches the request's end: sample from its last row


@dataclass
class StepPlan:
    entries: List[PlannedEntry] = field(default_factory=list)
    preempted: List[str] = field(default_factory=list)
    failed: List[str] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(len(e.tokens) for e in self.entries)


class Scheduler:
    def __init__(self, cache, max_num_seqs: int, max_num_batched_tokens: int, max_model_len: int,
                 max_prefill_portion: Optional[int] = None):
        if max_num_seqs < 1:
            raise SchedulerError("max_num_seqs must be >= 1")
        if max_num_batched_tokens < 1:
            raise SchedulerError("max_num_batched_tokens must be >= 1")
        if max_model_len < 1:
            raise SchedulerError("max_model_len must be >= 1")
        if max_prefill_portion is not None and max_prefill_portion < 1:
            raise SchedulerError("max_prefill_portion must be >= 1")
        self.cache = cache
        self.max_num_seqs = min(max_num_seqs, cache.max_requests)
        self.max_num_batched_tokens = max_num_batched_tokens
        self.max_model_len = max_model_len
        self.max_prefill_portion = max_prefill_portion
        self._requests: Dict[str, Request] = {}
        self._waiting: Deque[str] = deque()
        self._running: List[str] = []          # in admission order
        self._admissions = 0
        self.num_preemptions = 0

    # ------------------------------------------------------------------ admission
    def add_request(self, req: Request) -> None:
        """Queue the request, or record it as REJECTED (still observable through
        ``get_request``) when it can never run.  A duplicate id raises, as in the
        reference (scheduler.py:40-41)."""
        if req.request_id in self._requests:
            raise SchedulerError(f"duplicate request_id: {req.request_id}")
        self._requests[req.request_id] = req
        limit = self.max_model_len if req.context_limit is None else min(req.context_limit, self.max_model_len)
        n = len(req.prompt_token_ids)
        problem = req.sampling_params.problem()
        if problem is None and n == 0:
            problem = "empty prompt"
        if problem is None and n > limit:
            problem = f"prompt length {n} exceeds context limit {limit}"
        if problem is None and n + req.sampling_params.max_tokens > limit:
            problem = f"prompt length {n} + max_tokens {req.sampling_params.max_tokens} exceeds context limit {limit}"
        if problem is not None:
            req.error = problem
            req.transition(RequestState.REJECTED)
            return
        req.state = RequestState.WAITING
        self._waiting.append(req.request_id)

    def get_request(self, request_id: str) -> Request:
        return self._requests[request_id]

    @property
    def is_idle(self) -> bool:
        return not (self._waiting or self._running)

    @property
    def num_waiting(self) -> int:
        return len(self._waiting)

    @property
    def num_running(self) -> int:
        return len(self._running)

    # ------------------------------------------------------------------ ends of a request's life
    def _release(self, req: Request) -> None:
        if self.cache.has_request(req.request_id):
            self.cache.free_request(req.request_id)
        if req.request_id in self._running:
            self._running.remove(req.request_id)

    def cancel(self, request_id: str) -> None:
        req = self._requests.get(request_id)
        if req is None or req.is_terminal():
            return
        self._release(req)
        self._waiting = deque(r for r in self._waiting if r != request_id)
        req.transition(RequestState.CANCELLED)

    def finish(self, request_id: str, reason: str) -> None:
        req = self._requests.get(request_id)
        if req is None or req.is_terminal():
            return
        self._release(req)
        req.finish_reason = reason
        req.transition(RequestState.FINISHED)

    def fail(self, request_id: str, error: str) -> None:
        req = self._requests.get(request_id)
        if req is None or req.is_terminal():
            return
        self._release(req)
        self._waiting = deque(r for r in self._waiting if r != request_id)
        req.error = error
        req.transition(RequestState.FAILED)

    def _preempt(self, req: Request, plan: StepPlan) -> None:
        self._release(req)
        req.num_computed_tokens = 0
        req.num_preemptions += 1
        self.num_preemptions += 1
        req.transition(RequestState.WAITING)
        self._waiting.appendleft(req.request_id)
        plan.preempted.append(req.request_id)

    # ------------------------------------------------------------------ planning one step
    def _tokens_that_fit(self, rid: str, want: int, reserved: List[int]) -> int:
        """The largest n <= want for which every group has the pages, given ``reserved``."""
        lo, hi = 0, want
        while lo < hi:
            mid = (lo + hi + 1) // 2
            if self.cache.can_allocate(rid, mid, reserved):
                lo = mid
            else:
                hi = mid - 1
        return lo

    def _reserve(self, rid: str, n: int, reserved: List[int]) -> None:
        for i, p in enumerate(self.cache.pages_needed(rid, n)):
            reserved[i] += p

    def schedule(self) -> StepPlan:
        plan = StepPlan()
        budget = self.max_num_batched_tokens
        reserved = [0] * len(self.cache.free_pages())
        planned = set()

        # 1. one token for every decoding request; preempt from the back when a page is missing
        i = 0
        while i < len(self._running):
            rid = self._running[i]
            req = self._requests[rid]
            if req.state is not RequestState.DECODING:
                i += 1
                continue
            if budget < 1:
                break
            while not self.cache.can_allocate(rid, 1, reserved):
                victim = self._requests[self._running[-1]]
                if victim.request_id == rid and len(self._running) == 1:
                    self.fail(rid, "out of KV pages")
                    plan.failed.append(rid)
                    break
                if victim.request_id in planned:      # cannot happen: victims come from the back
                    raise SchedulerError("a planned request would be preempted")
                self._preempt(victim, plan)
                if victim.request_id == rid:
                    break
            if rid not in self._running:
                continue                                # it failed or preempted itself; same index, next request
            self._reserve(rid, 1, reserved)
            plan.entries.append(PlannedEntry(rid, req.num_computed_tokens,
                                             (req.all_token_ids[req.num_computed_tokens],), True))
            planned.add(rid)
            budget -= 1
            i += 1

        # 2. portions for requests in prefill, oldest first
        for rid in list(self._running):
            req = self._requests[rid]
            if req.state is not RequestState.PREFILLING or budget < 1:
                continue
            budget -= self._plan_portion(req, budget, reserved, plan)
            planned.add(rid)

        # 3. admit from the head of the queue (not in a step that had to preempt: the pages a
        #    victim gave back are for those that stayed)
        while not plan.preempted and self._waiting and budget >= 1 and len(self._running) < self.max_num_seqs \
                and self.cache.num_free_slots > 0:
            rid = self._waiting[0]
            req = self._requests[rid]
            self.cache.add_request(rid)
            want = min(req.num_tokens, budget, self.max_prefill_portion or budget)
            if self._tokens_that_fit(rid, want, reserved) < 1:
                self.cache.free_request(rid)
                break
            self._waiting.popleft()
            self._admissions += 1
            req.admission_index = self._admissions
            req.transition(RequestState.PREFILLING)
            self._running.append(rid)
            budget -= self._plan_portion(req, budget, reserved, plan)

        # nothing can move although requests are running: the pool is too small for the oldest
        if not plan.entries and self._running:
            if len(self._running) > 1:
                self._preempt(self._requests[self._running[-1]], plan)
            else:
                rid = self._running[0]
                self.fail(rid, "out of KV pages")
                plan.failed.append(rid)
        elif not plan.entries and self._waiting and not self._running:
            rid = self._waiting.popleft()               # the head does not fit an empty pool
            self.fail(rid, "out of KV pages")
            plan.failed.append(rid)
        return plan

    def _plan_portion(self, req: Request, budget: int, reserved: List[int], plan: StepPlan) -> int:
        rest = req.num_tokens - req.num_computed_tokens
        want = min(rest, budget, self.max_prefill_portion or budget)
        n = self._tokens_that_fit(req.request_id, want, reserved)
        if n < 1:
            return 0
        self._reserve(req.request_id, n, reserved)
        s = req.num_computed_tokens
        plan.entries.append(PlannedEntry(req.request_id, s, tuple(req.all_token_ids[s:s + n]), n == rest))
        return n

    # ------------------------------------------------------------------ after the step ran
    def advance(self, entry: PlannedEntry) -> None:
        """The entry's tokens are stored: move the request's progress."""
        req = self._requests[entry.request_id]
        req.num_computed_tokens += len(entry.tokens)

    def on_token(self, request_id: str) -> None:
        """A token was sampled for the request: from now on it decodes."""
        req = self._requests[request_id]
        if req.state is RequestState.PREFILLING:
            req.transition(RequestState.DECODING)
