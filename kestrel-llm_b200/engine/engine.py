"""The engine: a model, its cache, and ONE step function.

``step(entries)`` takes a batch of (request, its next tokens) - portions of prompts beside
single decoded tokens, cut anywhere - reserves pages, runs exactly these tokens through the
model from the cache that earlier steps left, commits the cache, and returns the float32
logits at the wanted places.  The reference has three separate forward entry points
(src/model/vllm_safetensors.c:16356 single token, :17926 one request's prompt, :17041 one
token of each of n requests) and never mixes them; this one function covers all three and
their mixtures.  Generation (`LLM`), trace replay (`bin/trace_run`) and the benchmark all
call it.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager, OutOfPages
from ..config.engine_options import EngineOptions
from ..csrc import ops
from .batch import Entry, StepBatch


class Engine:
    def __init__(self, model, options: EngineOptions):
        self.model = model
        self.options = options
        dev = model.device
        if dev.type != "cuda":
            raise RuntimeError(f"the engine runs on a CUDA device, not on '{dev}': there is no CPU path")
        arch = ops.device_arch()
        if arch < 100:
            raise RuntimeError(f"this engine is written for sm_100a (B200); the device reports sm_{arch}")
        cfg = model.config
        self.max_model_len = options.max_model_len or cfg.max_position_embeddings
        page = options.page_size
        if options.num_pages:
            num_pages = options.num_pages
        elif options.max_tokens:
            num_pages = (options.max_tokens + page - 1) // page
        else:
            num_pages = self._pages_that_fit(model, options, page)
        self.cache = CacheManager(model.cache_specs(), model.dtype, dev, page, num_pages,
                                  options.batch_max, self.max_model_len)
        self.vocab_size = model.vocab_size
        self.graphs = None
        if options.cuda_graphs and getattr(model, "graph_safe", False):
            from .graphs import DecodeGraphs
            self.graphs = DecodeGraphs(model, self.cache, options.batch_max)
        # Steps that are not replayed from a graph run from the model's step program, one native
        # call a step, if every part of the model wrote itself into one; else by the parts' forward.
        self.runner = None
        if options.native_step and hasattr(model, "step_program"):
            program = model.step_program(self.cache)
            if program is not None:
                from .runner import StepRunner
                self.runner = StepRunner(program, self.cache, options.max_step_tokens, options.batch_max,
                                         guards=options.debug_guards)
        self.profile = None
        if options.profile:
            from .profile import PhaseProfile
            self.profile = PhaseProfile()
        self.steps_run = 0
        self.graph_launches = 0      # kernels replayed from CUDA graphs (not counted by ops.launches)
        self.native_launches = 0     # kernels launched by the native runner (not counted by ops.launches)
        self.last_h2d_bytes = 0

    def _pages_that_fit(self, model, options: EngineOptions, page: int) -> int:
        """Pages per cache group when no size is given: what the chosen share of the device's free
        memory holds (the weights are loaded already), at most batch_max requests of
        max_model_len tokens; the choice is printed."""
        import sys
        from ..parts.base import PagedKVSpec
        want = options.batch_max * self.max_model_len
        esize = torch.empty((), dtype=model.dtype).element_size()
        per_token = sum(2 * sp.kv_heads * sp.head_dim * esize for sp in model.cache_specs() if isinstance(sp, PagedKVSpec))
        if per_token == 0:
            return max(1, (want + page - 1) // page)
        free, _total = torch.cuda.mem_get_info(model.device)
        # room for activations of the largest step beside the cache
        reserve = 2 << 30
        fit = int(max(0, free * options.memory_fraction - reserve) // per_token)
        tokens = min(want, fit)
        if tokens < self.max_model_len:
            raise RuntimeError(f"the device has room for a cache of {fit} tokens ({per_token} bytes a token), less than one "
                               f"request of max_model_len {self.max_model_len}; lower max_model_len")
        if tokens < want:
            print(f"[kestrel] cache: {tokens} tokens ({tokens * per_token / 2**30:.1f} GiB) fit the device's free memory; "
                  f"{options.batch_max} requests of {self.max_model_len} tokens would need {want}", file=sys.stderr, flush=True)
        return (tokens + page - 1) // page

    # ---- requests -----------------------------------------------------------------------
    def admit(self, rid: int) -> int:
        """Gives a new request its state slot."""
        return self.cache.admit(rid)

    def release(self, rid: int) -> None:
        """Ends a request: its pages and its slot are given back."""
        self.cache.release(rid)

    # ---- the step -----------------------------------------------------------------------
    def step(self, entries: Sequence[Entry], reserved: bool = False, checked: bool = False,
             token_ids_dev: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Runs one batch.  Unknown requests are admitted.  Returns float32 logits
        [number of wanted places, vocab] on the device, in the order of entries and of each
        entry's ``want``; None if nothing was wanted.  If pages run out, `OutOfPages` is raised
        before anything runs; no request's length changes (pages that earlier entries of
        the same call had reserved stay with those requests for their next step).
        ``reserved``: the caller has reserved the pages already; ``checked``: it has checked that
        every token id lies inside the vocabulary.  ``token_ids_dev`` (int32 on the device, one id
        per entry; decode-only steps of a captured model) stands for the entries' token ids when
        the host does not know them yet: the ids the previous step sampled."""
        entries = [e for e in entries if len(e.tokens) > 0]
        if not entries:
            return None
        seen = set()
        for e in entries:
            if e.rid in seen:
                raise ValueError(f"request {e.rid} appears twice in one step")
            seen.add(e.rid)
            for w in e.want:
                if not 0 <= int(w) < len(e.tokens):
                    raise ValueError(f"request {e.rid}: wanted place {w} outside its {len(e.tokens)} tokens of this step")
            if checked:             # the caller vouches for the ids (prompts checked on arrival, ids it sampled itself)
                continue
            ids = np.asarray(e.tokens, dtype=np.int64)
            if ids.min() < 0 or ids.max() >= self.vocab_size:
                bad = int(ids[(ids < 0) | (ids >= self.vocab_size)][0])
                raise ValueError(f"request {e.rid}: token id {bad} outside the vocabulary of {self.vocab_size}")
        admitted: List[int] = []
        try:
            for e in entries:
                if not self.cache.is_live(e.rid):
                    self.cache.admit(e.rid)
                    admitted.append(e.rid)
                if self.cache.length(e.rid) + len(e.tokens) > self.max_model_len:
                    raise ValueError(f"request {e.rid} would grow beyond max_model_len {self.max_model_len}")
            if not reserved:
                for e in entries:
                    self.cache.reserve(e.rid, len(e.tokens))
        except Exception:
            for rid in admitted:
                self.cache.release(rid)
            raise
        self.cache.clear_admitted()       # state slots of requests admitted since the last step, by whomever
        decode_only = self.graphs is not None and self.profile is None and all(len(e.tokens) == 1 for e in entries)
        if token_ids_dev is not None and not decode_only:
            raise ValueError("token ids on the device stand for one token per entry of a captured decode step")
        if decode_only:
            # decode tokens only: replay the captured step of this batch-size bucket
            logits, batch, replayed = self.graphs.run(entries, token_ids_dev)
            self.graph_launches += replayed
            self.last_h2d_bytes = batch.bytes_h2d
            if any(len(e.want) == 0 for e in entries):
                keep = [i for i, e in enumerate(entries) if len(e.want)]
                logits = logits[torch.tensor(keep, dtype=torch.long, device=logits.device)] if keep else None
        elif self.runner is not None:
            logits = self.runner.step(entries, self.vocab_size, profile=self.profile)
            self.native_launches += self.runner.last_launches
            self.last_h2d_bytes = self.runner.last_h2d_bytes
        else:
            batch = StepBatch(entries, self.cache, self.model.device)
            logits = self.model.forward(batch, self.cache)
            self.last_h2d_bytes = batch.bytes_h2d
        for e in entries:
            self.cache.commit(e.rid, len(e.tokens))
        self.steps_run += 1
        return logits
