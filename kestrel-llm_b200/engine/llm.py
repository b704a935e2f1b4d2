"""The Python entry point: token ids in, token ids out.

    llm = LLM("/path/to/model", dtype="bfloat16")
    outs = llm.generate([[1, 2, 3], [4, 5]], SamplingParams(temperature=0.0, max_tokens=16))

The reference's request loop prefills a prompt, then samples and feeds one token at a time
until a stop token or the token limit (src/serve/vllm_server.c:1130-1595, 1595-1790; batching
src/serve/vllm_batch.c:303-493).  Here the scheduler builds mixed steps, every step is one
call of `Engine.step`, and tokens are picked on the device; per step the host sends the
step's description and reads back one token id per request that produced one.

Decode steps run ahead of the host: when every running request is decoding and nothing waits,
`step` launches the next step BEFORE it has read the ids the last one sampled - those go from the
sampler's output to the next step's input on the device - and reads them while the new step
runs.  A stop token is therefore seen one step late: the stopped request has one more token
computed, which is thrown away, and its pages are given back then.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Union

import torch

from ..config.engine_options import EngineOptions
from ..csrc import ops
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from ..weights.loader import load_model
from .batch import Entry
from .engine import Engine
from .scheduler import Scheduler


@dataclass
class RequestMetrics:
    """The six numbers the reference reports per request (VLLMMetrics,
    include/serve/vllm_server.h:322-339, filled in src/serve/vllm_batch.c:419-426): wall-clock
    milliseconds from the moment the request was added."""
    prompt_tokens: int = 0
    n_tokens: int = 0           # generated tokens
    prefill_ms: float = 0.0     # start -> the step that finished the prompt has run
    ttft_ms: float = 0.0        # start -> first token on the host
    tpot_ms: float = 0.0        # mean time per token after the first
    total_ms: float = 0.0       # start -> last token on the host


@dataclass
class RequestOutput:
    request_id: int
    prompt_token_ids: List[int]
    token_ids: List[int] = field(default_factory=list)
    finish_reason: Optional[str] = None       # "stop" | "length", as the reference reports them
    preemptions: int = 0
    metrics: RequestMetrics = field(default_factory=RequestMetrics)


@dataclass
class _Live:
    out: RequestOutput
    params: SamplingParams
    seed: int
    stop_ids: frozenset
    sampled: int = 0            # tokens sampled so far, those the host has not read yet included
    t_start: float = 0.0        # perf_counter when the request was added
    t_first: float = 0.0        # ... when its first token reached the host


@dataclass
class _InFlight:
    """A step whose sampled ids are still on their way to the host."""
    lives: List[_Live]
    ids_dev: torch.Tensor       # int32 [len(lives)] on the device
    ids_host: torch.Tensor      # pinned; filled when `done` has passed
    done: torch.cuda.Event
    decode_only: bool           # every entry of the step was a single decode token
    counted: bool = False       # the scheduler already counts these tokens
    discard: set = field(default_factory=set)      # requests that ended before this step's token was read


@dataclass
class StepStats:
    steps: int = 0
    prompt_tokens: int = 0
    generated_tokens: int = 0
    h2d_bytes: int = 0
    d2h_bytes: int = 0
    seconds: float = 0.0


@dataclass
class StepRecord:
    """One step as `LLM.record_steps` keeps it: what ran, and CUDA events around its kernels
    (their distance is the step's time on the device; the distance between the starts of
    consecutive steps holds the host's share too)."""
    tokens: int
    requests: int
    decode_only: bool
    start: torch.cuda.Event
    end: torch.cuda.Event


class LLM:
    def __init__(self, model: Union[str, object], dtype: str = "bfloat16",
                 options: Optional[EngineOptions] = None, **kw):
        """``model``: a folder with config.json and safetensors, or a model already built.
        Keyword arguments override fields of `EngineOptions` (page_size, batch_max ...)."""
        opts = options or EngineOptions()
        opts.dtype = dtype
        for k, v in kw.items():
            if not hasattr(opts, k):
                raise TypeError(f"unknown engine option '{k}'")
            setattr(opts, k, v)
        self.options = opts
        if isinstance(model, str):
            model = load_model(model, opts.normalised_dtype(), opts.device)
        self.model = model
        self.engine = Engine(model, opts)
        self.scheduler = Scheduler(self.engine.cache, opts.max_step_tokens, opts.prefill_batch,
                                   opts.batch_max, opts.max_queued, self.engine.max_model_len)
        self.sampler = Sampler(model.device)
        self._live: Dict[int, _Live] = {}
        self._next_id = 0
        self.stats = StepStats()
        self._ahead: Optional[_InFlight] = None
        self._pinned = [torch.empty(opts.batch_max + 8, dtype=torch.int32).pin_memory() for _ in range(3)]
        self._pinned_turn = 0
        self.run_ahead = not opts.profile   # False: every step's ids are read before the next step is built
        self.record_steps = False       # True: every step leaves a `StepRecord` in `step_records`
        self.step_records: List[StepRecord] = []

    # ---- requests -----------------------------------------------------------------------
    def add_request(self, prompt_token_ids: Sequence[int], params: Optional[SamplingParams] = None,
                    request_id: Optional[int] = None) -> int:
        params = params or SamplingParams()
        rid = self._next_id if request_id is None else request_id
        self._next_id = max(self._next_id, rid) + 1
        prompt = [int(t) for t in prompt_token_ids]
        for t in prompt:
            if not 0 <= t < self.engine.vocab_size:
                raise ValueError(f"token id {t} outside the vocabulary of {self.engine.vocab_size}")
        self.scheduler.add(rid, len(prompt), params.max_tokens)
        stop = set(params.stop_token_ids)
        if not params.ignore_eos:
            stop |= set(self.model.config.eos_token_ids)
        seed = params.seed if params.seed is not None else (self.options.seed * 1000003 + rid)
        lv = _Live(RequestOutput(rid, prompt), params, seed, frozenset(stop), t_start=time.perf_counter())
        lv.out.metrics.prompt_tokens = len(prompt)
        self._live[rid] = lv
        return rid

    def abort_request(self, rid: int) -> Optional[RequestOutput]:
        """Ends a request now, whatever its state; its pages and slot are given back."""
        lv = self._live.pop(rid, None)
        if lv is None:
            return None
        if self._ahead is not None:
            self._ahead.discard.add(rid)
        self.scheduler.finish(rid)
        lv.out.finish_reason = "abort"
        return lv.out

    def warm_up(self) -> int:
        """What a server does once before it takes requests: captures the decode step of every
        batch-size bucket and class of context now, so that no request waits for a capture.
        Returns the number of steps captured (0 if the model's steps are not captured)."""
        if self.engine.graphs is None:
            return 0
        n = self.engine.graphs.capture_all(self.engine.max_model_len)
        torch.cuda.synchronize(self.model.device)
        return n

    def has_unfinished(self) -> bool:
        return bool(self._live)

    # ---- one step -----------------------------------------------------------------------
    def step(self) -> List[RequestOutput]:
        """Schedules and runs one step; returns the requests found finished in this call (a
        decode step's tokens are read during the next call, see the module text)."""
        prev, self._ahead = self._ahead, None
        if prev is not None and self._can_run_ahead(prev):
            return self._step_ahead(prev)
        finished = self._finalize(prev, None) if prev is not None else []
        plan = self.scheduler.schedule()
        for rid in self.scheduler.preempted():
            self._live[rid].out.preemptions += 1
            self._live[rid].sampled = len(self._live[rid].out.token_ids)
        if not plan:
            return finished
        entries, sampling = [], []
        for s in plan:
            lv = self._live[s.rid]
            prompt, n_prompt = lv.out.prompt_token_ids, len(lv.out.prompt_token_ids)
            if s.start >= n_prompt:                   # a decode token (or recomputed output): no copy of the prompt
                piece = lv.out.token_ids[s.start - n_prompt:s.start - n_prompt + s.count]
            else:
                piece = prompt[s.start:s.start + s.count]
                if s.start + s.count > n_prompt:
                    piece = piece + lv.out.token_ids[:s.start + s.count - n_prompt]
            entries.append(Entry(s.rid, piece, (s.count - 1,) if s.wants_token else ()))
            if s.wants_token:
                sampling.append(lv)
            if s.start < n_prompt:
                self.stats.prompt_tokens += min(s.start + s.count, n_prompt) - s.start
        rec = self._begin_record(sum(s.count for s in plan), len(plan), all(s.count == 1 for s in plan))
        logits = self.engine.step(entries, reserved=True, checked=True)    # prompts were checked on arrival
        self.scheduler.step_done()
        self.stats.steps += 1
        self.stats.h2d_bytes += self.engine.last_h2d_bytes
        if sampling:
            decode_only = all(s.count == 1 and s.wants_token for s in plan)
            flight = self._sample(logits, sampling, decode_only)
            self._end_record(rec)
            if decode_only and self.run_ahead and self.engine.graphs is not None:
                self._ahead = flight            # read while the next step runs
            else:
                finished += self._finalize(flight, None)
        else:
            self._end_record(rec)
        return finished

    def _begin_record(self, tokens: int, requests: int, decode_only: bool) -> Optional[StepRecord]:
        if not self.record_steps:
            return None
        rec = StepRecord(tokens, requests, decode_only, torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        rec.start.record()
        return rec

    def _end_record(self, rec: Optional[StepRecord]) -> None:
        if rec is not None:
            rec.end.record()
            self.step_records.append(rec)

    def cache_occupancy(self) -> Dict[str, object]:
        """Pages of every cache group in use, and live requests: what the reference's serving
        loop watches as free memory before it admits (src/serve/vllm_server.c:82-101)."""
        c = self.engine.cache
        groups = [{"window": g.window, "pages": c.num_pages(i), "free": c.free_pages(i)} for i, g in enumerate(c.groups)]
        return {"page_size": c.page_size, "groups": groups, "live_requests": c.live_requests(),
                "running": self.scheduler.num_running, "waiting": self.scheduler.num_waiting}

    def _sample(self, logits: torch.Tensor, lives: List[_Live], decode_only: bool) -> _InFlight:
        """Picks one token per request on the device and starts their copy to the host."""
        ids_dev = self.sampler.sample(logits, [lv.params for lv in lives], [lv.seed for lv in lives],
                                      [lv.sampled for lv in lives], [lv.out.token_ids for lv in lives])
        for lv in lives:
            lv.sampled += 1
        host = self._pinned[self._pinned_turn]
        self._pinned_turn = (self._pinned_turn + 1) % len(self._pinned)
        host[:len(lives)].copy_(ids_dev, non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        self.stats.d2h_bytes += 4 * len(lives)
        return _InFlight(lives, ids_dev, host, done, decode_only)

    def _finalize(self, flight: _InFlight, newer: Optional[_InFlight]) -> List[RequestOutput]:
        """Waits for a step's ids, appends them and ends the requests that are over; a request
        that ends is struck from ``newer``, the step launched after this one."""
        flight.done.synchronize()
        ids = flight.ids_host[:len(flight.lives)].tolist()          # the step's only read-back: one id per request
        finished: List[RequestOutput] = []
        for lv, tok in zip(flight.lives, ids):
            rid = lv.out.request_id
            if rid in flight.discard or self._live.get(rid) is not lv:
                continue
            lv.out.token_ids.append(int(tok))
            self.stats.generated_tokens += 1
            now = time.perf_counter()
            m = lv.out.metrics
            if lv.t_first == 0.0:
                lv.t_first = now
                m.prefill_ms = m.ttft_ms = (now - lv.t_start) * 1000.0
            m.n_tokens = len(lv.out.token_ids)
            m.total_ms = (now - lv.t_start) * 1000.0
            m.tpot_ms = (now - lv.t_first) * 1000.0 / (m.n_tokens - 1) if m.n_tokens > 1 else m.ttft_ms
            at_limit = False if flight.counted else self.scheduler.on_token(rid)
            if int(tok) in lv.stop_ids:
                lv.out.finish_reason = "stop"
            elif at_limit or len(lv.out.token_ids) >= lv.params.max_tokens:
                lv.out.finish_reason = "length"
            if lv.out.finish_reason:
                self.scheduler.finish(rid)
                finished.append(lv.out)
                del self._live[rid]
                if newer is not None:
                    newer.discard.add(rid)
        return finished

    def _can_run_ahead(self, prev: _InFlight) -> bool:
        """Whether the step after ``prev`` is known without prev's ids: every running request
        decoded in prev and goes on for at least one more token, nothing waits, and pages for one
        more token of each are there (so that the scheduler preempts nobody)."""
        if not (self.run_ahead and prev.decode_only and self.engine.graphs is not None):
            return False
        if self.scheduler.num_waiting or self.scheduler.num_running != len(prev.lives):
            return False
        for lv in prev.lives:
            rid = lv.out.request_id
            if rid in prev.discard or self._live.get(rid) is not lv:
                return False
            if lv.sampled >= lv.params.max_tokens:           # the token in flight is its last
                return False
            if lv.params.penalised:                          # the penalty needs that token on the host
                return False
        cache = self.engine.cache
        return all(cache.free_pages(g) >= len(prev.lives) for g in range(cache.num_groups))

    def _step_ahead(self, prev: _InFlight) -> List[RequestOutput]:
        """Launches the next decode step on the ids ``prev`` left on the device, then reads them."""
        for lv in prev.lives:
            if self.scheduler.on_token(lv.out.request_id):
                raise RuntimeError("run-ahead: a request reached its token limit unexpectedly")
        prev.counted = True
        plan = self.scheduler.schedule()
        if [s.rid for s in plan] != [lv.out.request_id for lv in prev.lives] or \
                any(s.count != 1 or not s.wants_token for s in plan) or self.scheduler.preempted():
            raise RuntimeError("run-ahead: the scheduler built another step than the one foreseen")
        entries = [Entry(s.rid, (0,), (0,)) for s in plan]          # the ids are on the device
        rec = self._begin_record(len(plan), len(plan), True)
        logits = self.engine.step(entries, reserved=True, checked=True, token_ids_dev=prev.ids_dev)
        self.scheduler.step_done()
        self.stats.steps += 1
        self.stats.h2d_bytes += self.engine.last_h2d_bytes
        flight = self._sample(logits, prev.lives, True)
        self._end_record(rec)
        finished = self._finalize(prev, flight)
        self._ahead = flight if self._live else None                 # all ended: the extra tokens are dropped
        return finished

    # ---- whole runs ---------------------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]],
                 params: Union[SamplingParams, Sequence[SamplingParams], None] = None) -> List[RequestOutput]:
        """Generates for every prompt (lists of token ids); outputs in the order of prompts."""
        if params is None or isinstance(params, SamplingParams):
            plist = [params or SamplingParams()] * len(prompts)
        else:
            plist = list(params)
            if len(plist) != len(prompts):
                raise ValueError("one SamplingParams per prompt, or one for all")
        t0 = time.perf_counter()
        rids = [self.add_request(p, sp) for p, sp in zip(prompts, plist)]
        done = self.run_until_done()
        self.stats.seconds += time.perf_counter() - t0
        return [done[r] for r in rids]

    def run_until_done(self, on_step=None) -> Dict[int, RequestOutput]:
        """Steps until no request is left; returns the finished requests by id.  ``on_step`` is
        called after every step with the requests it found finished.  Raises if the scheduler
        finds nothing to run although requests are live, and if a kernel gave up a bounded wait
        (no tokens are better than wrong ones)."""
        done: Dict[int, RequestOutput] = {}
        idle = 0
        while self.has_unfinished():
            before = self.engine.steps_run
            fin = self.step()
            for o in fin:
                done[o.request_id] = o
            if on_step is not None:
                on_step(fin)
            if not fin and self.engine.steps_run == before:
                idle += 1
                if idle > 3:
                    raise RuntimeError("the scheduler found nothing to run although requests are waiting")
            else:
                idle = 0
        torch.cuda.synchronize(self.model.device)
        ops.raise_on_kernel_error()
        if self.engine.profile is not None and hasattr(self.engine.profile, "print_summary"):
            self.engine.profile.print_summary()
        return done
