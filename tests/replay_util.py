"""Helpers of the GPU tests: traces in the form `bin/trace_run` reads, an in-process runner
that feeds them to the engine's step function, and the comparison with the plain
implementation."""
from __future__ import annotations

import functools
import os
from typing import Dict, List, Sequence, Tuple

import numpy as np

import plain_qwen3 as P

# Largest allowed |engine - plain| as a fraction of the largest |plain logit| of the request.
# float32: rounding of float32 sums in another order.  bfloat16: activations and cache are
# rounded to 8 bits of mantissa between kernels.  These are not to be widened to make a test
# pass; a difference that shows in one way of cutting only is a fault of the cache or batch.
TOL = {"float32": 5e-6, "bfloat16": 2e-2}


@functools.lru_cache(maxsize=None)
def _plain_cached(model_dir: str, tokens: Tuple[int, ...]) -> np.ndarray:
    cfg, W = P.read_model(model_dir)
    return P.forward_logits(cfg, W, list(tokens))


def plain_logits(model_dir: str, tokens: Sequence[int]) -> np.ndarray:
    return _plain_cached(model_dir, tuple(int(t) for t in tokens))


def random_requests(vocab: int, lengths: Sequence[int], seed: int) -> Dict[str, List[int]]:
    rng = np.random.default_rng(seed)
    return {f"r{i}": rng.integers(0, vocab, size=n).tolist() for i, n in enumerate(lengths)}


def ceil64(n: int) -> int:
    return (n + 63) // 64 * 64


# ---- trace families --------------------------------------------------------------------------

def trace_whole(reqs: Dict[str, List[int]]):
    steps = []
    for name, toks in reqs.items():
        steps.append({"entries": [{"id": name, "tokens": toks, "want": list(range(len(toks)))}], "end": [name]})
    return steps, max(ceil64(len(t)) for t in reqs.values())


def trace_tail_decode(reqs: Dict[str, List[int]], tail: int = 32):
    steps = []
    for name, toks in reqs.items():
        head = max(1, len(toks) - tail) if len(toks) > tail else 1
        steps.append({"entries": [{"id": name, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        for i in range(head, len(toks)):
            steps.append({"entries": [{"id": name, "tokens": [toks[i]], "want": [0]}], "end": []})
        steps[-1]["end"] = [name]
    return steps, max(ceil64(len(t)) for t in reqs.values())


def trace_portions(reqs: Dict[str, List[int]], sizes=(7, 2, 13, 2, 5, 3, 17, 2, 31, 4)):
    steps = []
    k = 0
    for name, toks in reqs.items():
        pos = 0
        while pos < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - pos)
            if len(toks) - pos - n == 1:       # never leave a single token: portions go down to two
                n += 1
            k += 1
            steps.append({"entries": [{"id": name, "tokens": toks[pos:pos + n], "want": list(range(n))}], "end": []})
            pos += n
        steps[-1]["end"] = [name]
    return steps, max(ceil64(len(t)) for t in reqs.values())


def trace_mixed(reqs: Dict[str, List[int]], live_max: int = 4, tail: int = 12,
                sizes=(9, 2, 14, 3, 6, 2, 21, 5), seed: int = 0):
    """Up to `live_max` requests live at a time: portions of some beside single decoded tokens
    of others; a request may sit out a step; a finished request's pages are given back and the
    next request starts in a later step on those pages.  Returns (steps, max_tokens) with
    max_tokens = the most tokens held at any time, each live request's final length rounded up
    to 64 - the pool that `bin/trace_run --max-tokens` is made for."""
    rng = np.random.default_rng(seed)
    waiting = list(reqs.items())
    live: List[List] = []          # [name, toks, pos]
    steps = []
    k = 0
    peak = 0
    while waiting or live:
        while waiting and len(live) < live_max:
            name, toks = waiting.pop(0)
            live.append([name, toks, 0])
            if rng.random() < 0.5:
                break              # admit the others in later steps
        peak = max(peak, sum(ceil64(len(t)) for _, t, _ in live))
        entries, ends = [], []
        for item in live:
            name, toks, pos = item
            if len(live) > 1 and rng.random() < 0.2:
                continue           # left out of this step, goes on later
            left = len(toks) - pos
            if left > tail:
                n = min(sizes[k % len(sizes)], left - tail)
                k += 1
                if n < 2:
                    n = min(2, left)
            else:
                n = 1
            entries.append({"id": name, "tokens": toks[pos:pos + n], "want": list(range(n))})
            item[2] = pos + n
            if item[2] == len(toks):
                ends.append(name)
        if not entries:
            continue
        steps.append({"entries": entries, "end": ends})
        live = [it for it in live if it[2] < len(it[1])]
    return steps, peak


# ---- running a trace in-process ---------------------------------------------------------------

def make_engine(model_dir: str, dtype: str, max_tokens: int, page_size: int = 16, batch_max: int = 8,
                graphs: bool = False, native: bool = True, guards: bool = False):
    from kestrel_llm_b200.config import EngineOptions
    from kestrel_llm_b200.engine import Engine
    from kestrel_llm_b200.weights import load_model
    opts = EngineOptions(dtype=dtype, page_size=page_size, batch_max=batch_max,
                         num_pages=max(1, (max_tokens + page_size - 1) // page_size), cuda_graphs=graphs,
                         native_step=native, debug_guards=guards)
    model = load_model(model_dir, dtype, opts.device)
    return Engine(model, opts)


def run_trace(engine, steps) -> Dict[str, Dict[int, np.ndarray]]:
    """Feeds the steps to engine.step; returns {request: {position: logits row}}."""
    from kestrel_llm_b200.engine import Entry
    ids: Dict[str, int] = {}
    issued = 0
    pos: Dict[str, int] = {}
    out: Dict[str, Dict[int, np.ndarray]] = {}
    for st in steps:
        entries = []
        places = []
        for e in st["entries"]:
            if e["id"] not in ids:
                ids[e["id"]] = issued
                issued += 1
                pos[e["id"]] = 0
                out.setdefault(e["id"], {})
            entries.append(Entry(ids[e["id"]], e["tokens"], e["want"]))
            for w in e["want"]:
                places.append((e["id"], pos[e["id"]] + w))
            pos[e["id"]] += len(e["tokens"])
        logits = engine.step(entries)
        if logits is not None:
            arr = logits.float().cpu().numpy()
            assert arr.shape[0] == len(places)
            for (name, p), row in zip(places, arr):
                out[name][p] = row
        for name in st["end"]:
            engine.release(ids.pop(name))
            pos.pop(name)
        engine.cache.check()
    return out


def compare_with_plain(model_dir_f32: str, reqs: Dict[str, List[int]], got, dtype: str, label: str = ""):
    """Every logits row the trace produced against the plain implementation; returns the
    largest relative error seen.  On failure names the first wrong (request, position)."""
    tol = TOL[dtype]
    worst = 0.0
    for name, toks in reqs.items():
        ref = plain_logits(model_dir_f32, toks)
        scale = float(np.abs(ref).max())
        assert set(got[name]) == set(range(len(toks))), f"{label}: {name} misses positions"
        for p in range(len(toks)):
            row = got[name][p]
            assert np.isfinite(row).all(), f"{label}: {name} position {p}: logits are not finite"
            err = float(np.abs(row - ref[p]).max()) / scale
            worst = max(worst, err)
            assert err <= tol, (f"{label}: first wrong place: request {name} position {p} of {len(toks)}: "
                                f"error {err:.3e} of the largest logit, allowed {tol:.1e}")
    return worst
