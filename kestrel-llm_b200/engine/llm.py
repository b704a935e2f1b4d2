"""The Python entry point: token ids in, token ids out.

    llm = LLM("/path/to/model", dtype="bfloat16")
    outs = llm.generate([[1, 2, 3], [4, 5]], SamplingParams(temperature=0.0, max_tokens=16))

The reference's request loop prefills a prompt, then samples and feeds one token at a time
until a stop token or the token limit (src/serve/vllm_server.c:1130-1595, 1595-1790; batching
src/serve/vllm_batch.c:303-493).  Here the scheduler builds mixed steps, every step is one
call of `Engine.step`, and tokens are picked on the device; per step the host sends the
step's description and reads back one token id per request that produced one.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Union

import torch

from ..config.engine_options import EngineOptions
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from ..weights.loader import load_model
from .batch import Entry
from .engine import Engine
from .scheduler import Scheduler


@dataclass
class RequestOutput:
    request_id: int
    prompt_token_ids: List[int]
    token_ids: List[int] = field(default_factory=list)
    finish_reason: Optional[str] = None       # "stop" | "length", as the reference reports them
    preemptions: int = 0


@dataclass
class _Live:
    out: RequestOutput
    params: SamplingParams
    seed: int
    stop_ids: frozenset


@dataclass
class StepStats:
    steps: int = 0
    prompt_tokens: int = 0
    generated_tokens: int = 0
    h2d_bytes: int = 0
    d2h_bytes: int = 0
    seconds: float = 0.0


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
        self._live[rid] = _Live(RequestOutput(rid, prompt), params, seed, frozenset(stop))
        return rid

    def abort_request(self, rid: int) -> Optional[RequestOutput]:
        """Ends a request now, whatever its state; its pages and slot are given back."""
        lv = self._live.pop(rid, None)
        if lv is None:
            return None
        self.scheduler.finish(rid)
        lv.out.finish_reason = "abort"
        return lv.out

    def has_unfinished(self) -> bool:
        return bool(self._live)

    # ---- one step -----------------------------------------------------------------------
    def step(self) -> List[RequestOutput]:
        """Schedules and runs one step; returns the requests that finished in it."""
        plan = self.scheduler.schedule()
        for rid in self.scheduler.preempted():
            self._live[rid].out.preemptions += 1
        if not plan:
            return []
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
            if s.start < len(lv.out.prompt_token_ids):
                self.stats.prompt_tokens += min(s.start + s.count, len(lv.out.prompt_token_ids)) - s.start
        logits = self.engine.step(entries, reserved=True, checked=True)    # prompts were checked on arrival
        self.scheduler.step_done()
        self.stats.steps += 1
        self.stats.h2d_bytes += self.engine.last_batch.bytes_h2d
        finished: List[RequestOutput] = []
        if sampling:
            ids_dev = self.sampler.sample(logits, [lv.params for lv in sampling], [lv.seed for lv in sampling],
                                          [len(lv.out.token_ids) for lv in sampling])
            ids = ids_dev.cpu().tolist()          # the step's only read-back: one id per request
            self.stats.d2h_bytes += 4 * len(ids)
            for lv, tok in zip(sampling, ids):
                rid = lv.out.request_id
                lv.out.token_ids.append(int(tok))
                self.stats.generated_tokens += 1
                at_limit = self.scheduler.on_token(rid)
                if int(tok) in lv.stop_ids:
                    lv.out.finish_reason = "stop"
                elif at_limit or len(lv.out.token_ids) >= lv.params.max_tokens:
                    lv.out.finish_reason = "length"
                if lv.out.finish_reason:
                    self.scheduler.finish(rid)
                    finished.append(lv.out)
                    del self._live[rid]
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
        done: Dict[int, RequestOutput] = {}
        idle = 0
        while self.has_unfinished():
            fin = self.step()
            for o in fin:
                done[o.request_id] = o
            if not fin and self.engine.steps_run == 0:
                idle += 1
                if idle > 3:
                    raise RuntimeError("the scheduler found nothing to run although requests are waiting")
        torch.cuda.synchronize(self.model.device)
        self.stats.seconds += time.perf_counter() - t0
        return [done[r] for r in rids]
