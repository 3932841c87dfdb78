"""The engine: requests in, tokens out, one step at a time.

The shape is the reference's (src/infurnace/engine/engine.py:36-177): an offline request
API (``add_request``, ``add_text_request``, ``cancel``, ``output_tokens``, ``final_text``,
``metrics_of``, ``is_done``) around ``step() = commit_step(execute_step(prepare_step()))``.
What differs is inside a step: the plan is one mixed batch, run by one call of the step
function, and sampling happens on the device for all its rows at once.

Failures are contained as in the reference (engine.py:125-132,195-197): an exception from
the step function turns the requests of that step into FAILED ones, their pages and slots
go back, and the engine goes on with the others.  A fault that a kernel contained and
recorded on the device (a bounded wait that gave up, a token id outside the vocabulary) is
read every 32 steps and before any request is reported finished; it fails every request
that ran since the error word was last read clean.
"""
from __future__ import annotations

import time
import traceback
from dataclasses import dataclass, field
from typing import Dict, List, Mapping, Optional, Sequence, Tuple

from ..errors import KernelError, OutOfPages
from ..sampling import uniform
from ..tokenizer import StreamingDetokenizer, Tokenizer, check_stop_strings
from .loading import EngineOptions, build_runner
from .request import Request, RequestMetrics, RequestState, SamplingParams
from .runner import StepEntry
from .scheduler import PlannedEntry, Scheduler, StepPlan


@dataclass(frozen=True)
class EngineStepResult:
    """What one step did (the reference's fields, engine.py:13-21, and the step's counts)."""
    completed_requests: Tuple[str, ...] = ()
    new_tokens: Mapping[str, Tuple[int, ...]] = field(default_factory=dict)
    new_text: Mapping[str, str] = field(default_factory=dict)
    metrics: Mapping[str, RequestMetrics] = field(default_factory=dict)
    failed_requests: Tuple[str, ...] = ()
    preempted_requests: Tuple[str, ...] = ()
    num_prefill_tokens: int = 0
    num_decode_tokens: int = 0
    free_pages: Tuple[int, ...] = ()


@dataclass
class RawStep:
    """A step that was launched: its plan, and the sampled token ids on their way to the host."""
    plan: StepPlan
    handle: object = None                  # SampledTokens of the step (None: nothing was sampled)
    sampled: List[str] = field(default_factory=list)     # request ids, in the order of the handle's rows
    tokens: Dict[str, int] = field(default_factory=dict)
    error: Optional[str] = None


class Engine:
    def __init__(self, runner, scheduler: Optional[Scheduler] = None,
                 tokenizer: Optional[Tokenizer] = None, eos_token_ids: Sequence[int] = (), max_prefill_portion=None):
        self.runner = runner
        self.scheduler = scheduler or Scheduler(runner.cache, runner.max_requests, runner.max_tokens,
                                                runner.max_model_len, max_prefill_portion)
        self.tokenizer = tokenizer
        self.eos_token_ids = list(eos_token_ids)
        self._detoks: Dict[str, StreamingDetokenizer] = {}
        self._count = 0
        self._steps_since_check = 0
        self._ran_since_check: set = set()             # requests with a step launched since the error word was read clean
        self._inflight: Optional[RawStep] = None       # a step launched ahead of the one being committed
        self.overlap_decode = True

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_model_dir(cls, model_dir: str, options: Optional[EngineOptions] = None, tokenizer=None,
                       eos_token_ids: Sequence[int] = (), kernels=None, progress=None, **overrides) -> "Engine":
        """An engine for the model folder.  ``overrides`` are fields of :class:`EngineOptions`."""
        options = options or EngineOptions()
        for k, v in overrides.items():
            if not hasattr(options, k):
                raise TypeError(f"unknown engine option {k!r}")
            setattr(options, k, v)
        config, plan, runner = build_runner(model_dir, options, kernels=kernels, progress=progress)
        eng = cls(runner, tokenizer=tokenizer, eos_token_ids=eos_token_ids)
        eng.config, eng.plan, eng.options = config, plan, options
        return eng

    @classmethod
    def from_random(cls, config, seed: int, options: Optional[EngineOptions] = None, store_dtype="bfloat16",
                    workdir: Optional[str] = None, tokenizer=None, eos_token_ids: Sequence[int] = (), kernels=None,
                    progress=None, **overrides) -> "Engine":
        """Random weights for ``config`` (a typed configuration or a config.json mapping) from ``seed``.
        Without ``workdir`` the tensors are drawn on the device, no file is written, and a model of any
        size that fits the device can be made; with ``workdir`` a model folder is written there and
        loaded.  Both give the same tensors."""
        from ..models import config_from_dict
        if isinstance(config, Mapping):
            config = config_from_dict(config)
        if workdir is not None:
            from ..weights.random_init import write_random_model
            write_random_model(config, seed, workdir, store_dtype=store_dtype)
            return cls.from_model_dir(workdir, options, tokenizer=tokenizer, eos_token_ids=eos_token_ids, kernels=kernels,
                                      progress=progress, **overrides)
        options = options or EngineOptions()
        for k, v in overrides.items():
            if not hasattr(options, k):
                raise TypeError(f"unknown engine option {k!r}")
            setattr(options, k, v)
        config, plan, runner = build_runner(None, options, kernels=kernels, progress=progress,
                                            random=(config, seed, store_dtype))
        eng = cls(runner, tokenizer=tokenizer, eos_token_ids=eos_token_ids)
        eng.config, eng.plan, eng.options = config, plan, options
        return eng

    # ------------------------------------------------------------------ offline request API
    def add_request(self, req: Request) -> None:
        if not req.eos_token_ids and self.eos_token_ids:
            req.eos_token_ids = list(self.eos_token_ids)
        self.scheduler.add_request(req)

    def add_text_request(self, prompt: str, sampling_params: Optional[SamplingParams] = None,
                         stop_strings: Optional[List[str]] = None, request_id: Optional[str] = None,
                         context_limit: Optional[int] = None, **kw) -> Request:
        if self.tokenizer is None:
            raise RuntimeError("engine has no tokenizer; cannot add a text request")
        ids = self.tokenizer.encode(prompt)
        self._count += 1
        req = Request(request_id or f"req-{self._count}", ids, sampling_params or SamplingParams(), context_limit,
                      prompt=prompt, stop_strings=stop_strings or [], **kw)
        self._detoks[req.request_id] = StreamingDetokenizer(self.tokenizer, skip_prompt_len=len(ids))
        self.add_request(req)
        return req

    def cancel(self, request_id: str) -> None:
        self.scheduler.cancel(request_id)

    def output_tokens(self, request_id: str) -> Tuple[int, ...]:
        return self.scheduler.get_request(request_id).output_token_ids

    def metrics_of(self, request_id: str) -> RequestMetrics:
        return self.scheduler.get_request(request_id).metrics

    def final_text(self, request_id: str) -> str:
        d = self._detoks.get(request_id)
        return d.text if d else ""

    def is_done(self) -> bool:
        return self.scheduler.is_idle and self._inflight is None

    # ------------------------------------------------------------------ the three phases of a step
    def prepare_step(self) -> StepPlan:
        return self.scheduler.schedule()

    def execute_step(self, plan: StepPlan, feed=None, pending: int = 0) -> RawStep:
        """Launch the plan's step; nothing here waits for the device.  ``feed`` and ``pending`` are for a
        step that is launched while the one before it is still in flight (see ``step``): its input
        tokens come from the device, and each request's draw counter is ``pending`` ahead."""
        raw = RawStep(plan)
        if not plan.entries:
            return raw
        entries = [StepEntry(e.request_id, e.tokens, [len(e.tokens) - 1] if e.sample else []) for e in plan.entries]
        try:
            sampled = [e for e in plan.entries if e.sample]
            reqs = [self.scheduler.get_request(e.request_id) for e in sampled]
            temps = [r.sampling_params.effective_temperature for r in reqs]
            us = [uniform(r.sampling_params.seed, len(r.output_token_ids) + pending) if t > 0.0 else 0.0
                  for r, t in zip(reqs, temps)]
            raw.handle = self.runner.step_and_sample(entries, temps, us, feed=feed)
            raw.sampled = [e.request_id for e in sampled]
            for e in plan.entries:                 # the tokens' keys and values are in the pages now
                self.scheduler.advance(e)
                self._ran_since_check.add(e.request_id)
            self._steps_since_check += 1
        except Exception as e:  # a failed step fails its requests, not the engine
            if not isinstance(e, OutOfPages):
                traceback.print_exc()
            raw.error = f"{type(e).__name__}: {e}"
        return raw

    def commit_step(self, raw: RawStep) -> EngineStepResult:
        plan, sch = raw.plan, self.scheduler
        if raw.error is None and raw.handle is not None:
            raw.tokens = {rid: int(t) for rid, t in zip(raw.sampled, raw.handle.tolist())}
        completed, failed = [], list(plan.failed)
        new_tokens: Dict[str, List[int]] = {}
        new_text: Dict[str, str] = {}
        metrics: Dict[str, RequestMetrics] = {}
        finishing: List[Tuple[str, str]] = []
        n_prefill = n_decode = 0
        for e in plan.entries:
            req = sch.get_request(e.request_id)
            if req.is_terminal():        # cancelled or failed between the phases: its output is dropped
                continue
            if raw.error is not None:
                sch.fail(e.request_id, raw.error)
                failed.append(e.request_id)
                continue
            if req.state is RequestState.DECODING:
                n_decode += len(e.tokens)
            else:
                n_prefill += len(e.tokens)
            if not e.sample:
                continue
            tok = raw.tokens[e.request_id]
            req.append_output_token(tok)
            sch.on_token(e.request_id)
            new_tokens.setdefault(e.request_id, []).append(tok)
            reason = req.check_finished(tok)
            detok = self._detoks.get(e.request_id)
            delta = ""
            if detok is not None:
                delta = detok.update(req.all_token_ids)
                new_text[e.request_id] = new_text.get(e.request_id, "") + delta
            if reason is None and self.tokenizer is not None and self.tokenizer.is_end(tok):
                reason = "eos"
            if reason is None and detok is not None and req.stop_strings:
                hit, _s, keep = check_stop_strings(detok.text, req.stop_strings,
                                                   req.sampling_params.include_stop_str_in_output)
                if hit:
                    reason = "stop"
                    before = len(detok.text) - len(delta)
                    detok.truncate(keep)
                    new_text[e.request_id] = detok.text[before:]
            if reason is not None:
                finishing.append((e.request_id, reason))
        # reading the kernels' error word costs a device round trip: every 32 steps, and before a request is
        # reported finished (so that no request finishes on output that a kernel had marked invalid)
        if raw.error is None and (finishing or self._steps_since_check >= 32):
            failed.extend(self.contain_device_errors())
        for rid, reason in finishing:
            req = sch.get_request(rid)
            if req.is_terminal():
                continue
            sch.finish(rid, reason)
            metrics[rid] = req.metrics
            completed.append(rid)
        return EngineStepResult(
            completed_requests=tuple(completed), new_tokens={k: tuple(v) for k, v in new_tokens.items()},
            new_text=new_text, metrics=metrics, failed_requests=tuple(failed),
            preempted_requests=tuple(plan.preempted), num_prefill_tokens=n_prefill, num_decode_tokens=n_decode,
            free_pages=tuple(self.runner.cache.free_pages()))

    def step(self) -> EngineStepResult:
        """One step's results.  While requests only decode, the next step is launched before this
        one's tokens are read (``overlap_decode``): its input tokens are taken on the device from
        what this step sampled, so the host's share of a step (planning, staging, reading back)
        runs beside the device's.  A request that turns out to have stopped on this step's token
        has then computed one token too many, which is dropped with the request."""
        if self._inflight is None:
            self._inflight = self.execute_step(self.prepare_step())
        current, self._inflight = self._inflight, None
        if self.overlap_decode and current.error is None:
            ahead = self._plan_ahead(current)
            if ahead is not None:
                plan, rows = ahead
                self._inflight = self.execute_step(plan, feed=(current.handle, rows), pending=1)
        return self.commit_step(current)

    def _plan_ahead(self, current: RawStep):
        """The step after ``current`` if it is plain: every entry of ``current`` decoded one token, nobody
        waits, and each of those requests, unless this token is its last by count, decodes one more."""
        sch, cache = self.scheduler, self.runner.cache
        plan = current.plan
        if not plan.entries or plan.preempted or plan.failed or sch.num_waiting or current.handle is None:
            return None
        if len(plan.entries) != sch.num_running:
            return None
        entries, rows, reserved = [], [], [0] * len(cache.free_pages())
        for i, e in enumerate(plan.entries):
            req = sch.get_request(e.request_id)
            if len(e.tokens) != 1 or not e.sample or req.state is not RequestState.DECODING:
                return None
            sp = req.sampling_params
            produced = len(req.output_token_ids) + 1          # with the token that is on its way
            if produced >= sp.min_tokens and produced >= sp.max_tokens:
                continue                                       # it ends with that token, whatever it is
            if req.num_tokens + 1 >= self.runner.max_model_len or not cache.can_allocate(e.request_id, 1, reserved):
                return None
            for g, p in enumerate(cache.pages_needed(e.request_id, 1)):
                reserved[g] += p
            entries.append(PlannedEntry(e.request_id, req.num_computed_tokens, (-1,), True))
            rows.append(i)
        if not entries:
            return None
        return StepPlan(entries=entries), rows

    def check_device_errors(self) -> None:
        """Raise if a kernel recorded a fault since the error word was last read (a bounded wait on a
        barrier that gave up, a token id outside the vocabulary)."""
        self._steps_since_check = 0
        check = getattr(self.runner.rt.kernels, "check_device_errors", None)
        if check is not None:
            check()
        self._ran_since_check.clear()

    def contain_device_errors(self) -> List[str]:
        """Read the kernels' error word; if it is set, every request that had a step launched since it
        was last read clean FAILS (pages and state slot back, the error as its ``error``), as a runner
        exception fails the requests of its step (src/infurnace/engine/engine.py:125-132).  Returns the
        ids of the requests that failed.  A step launched ahead for them is dropped at its commit."""
        try:
            self.check_device_errors()
            return []
        except KernelError as err:
            failed = []
            for rid in sorted(self._ran_since_check):
                req = self.scheduler.get_request(rid)
                if not req.is_terminal():
                    self.scheduler.fail(rid, f"KernelError: {err}")
                    failed.append(rid)
            self._ran_since_check.clear()
            return failed

    # ------------------------------------------------------------------ conveniences
    def generate(self, prompts: Sequence[Sequence[int]], sampling_params=None) -> List[List[int]]:
        """Token ids in, generated token ids out, for a list of prompts (one
        :class:`SamplingParams` for all, or one per prompt)."""
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params or SamplingParams()] * len(prompts)
        ids = []
        for p, sp in zip(prompts, sampling_params):
            self._count += 1
            rid = f"gen-{self._count}"
            ids.append(rid)
            self.add_request(Request(rid, list(p), sp))
        idle_steps = 0
        while not self.is_done():
            res = self.step()
            moved = res.num_prefill_tokens or res.num_decode_tokens or res.failed_requests or res.preempted_requests
            idle_steps = 0 if moved else idle_steps + 1
            if idle_steps > 100:
                raise RuntimeError("the scheduler made no progress in 100 steps")
        self.contain_device_errors()
        out = []
        for rid in ids:
            req = self.scheduler.get_request(rid)
            if req.state is not RequestState.FINISHED:
                raise RuntimeError(f"request {rid} ended {req.state.value}: {req.error}")
            out.append(list(req.output_token_ids))
        return out


def generate(engine: Engine, prompt: Sequence[int], max_tokens: int):
    """One prompt, greedy, with timings: ``(all token ids, timings_ms)`` in the manner of the
    reference's tool (tools/run_infurnace_model.py:19-44): ``prefill_ms`` up to the first
    token, then ``first_decode_ms``, ``avg_decode_ms`` and ``decode_times_ms`` per token."""
    engine._count += 1
    rid = f"run-{engine._count}"
    engine.add_request(Request(rid, list(prompt), SamplingParams(max_tokens=max(1, max_tokens))))
    req = engine.scheduler.get_request(rid)
    if req.state is RequestState.REJECTED:
        raise ValueError(req.error)
    timings: Dict[str, object] = {}
    decode_times: List[float] = []
    t0 = time.perf_counter()
    while not req.is_terminal():
        had = len(req.output_token_ids)
        engine.step()
        if len(req.output_token_ids) > had:
            dt = (time.perf_counter() - t0) * 1000
            if had == 0:
                timings["prefill_ms"] = dt
            else:
                decode_times.append(dt)
            t0 = time.perf_counter()
    while not engine.is_done():            # a step launched ahead for the finished request
        engine.step()
    if req.state is not RequestState.FINISHED:
        raise RuntimeError(f"generation ended {req.state.value}: {req.error}")
    if decode_times:
        timings["first_decode_ms"] = decode_times[0]
        timings["avg_decode_ms"] = sum(decode_times) / len(decode_times)
        timings["decode_times_ms"] = decode_times
    return list(req.all_token_ids), timings
