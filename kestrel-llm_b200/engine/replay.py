"""Trace replay: given token ids, step by step, through the engine's own step function.

Nothing here computes: `Engine.step` is the model, cache and kernels that generation uses.
One JSON object a line on standard input:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which logits are wanted, ``<out>/<step>.f32`` gets them as little-endian float32
[wanted, vocab] in the order of the entries and of each ``want``.  After every step
``done <step>`` is printed and flushed.  The reference's nearest tools compare two arms of
its own harness by hashes (src/main.c:3326-3338, src/model/vllm_safetensors.c:16310-16354);
none of them takes a trace or writes logits.
"""
from __future__ import annotations

import json
import os
import sys


def replay_stdin(model_dir: str, dtype: str, out_dir: str, max_tokens: int, page_size: int = 16,
                 stream=None, cuda_graphs: bool = False) -> int:
    """``cuda_graphs``: steps of one token per request replay captured graphs, as generation's
    decode steps do; off, every step launches its kernels one by one (the same kernels)."""
    import torch

    from ..config import EngineOptions
    from ..csrc import ops
    from ..weights import load_model
    from .batch import Entry
    from .engine import Engine

    stream = stream or sys.stdin
    os.makedirs(out_dir, exist_ok=True)
    opts = EngineOptions(dtype=dtype, page_size=page_size, batch_max=8,
                         num_pages=max(1, (max_tokens + page_size - 1) // page_size), cuda_graphs=cuda_graphs)
    dtype = opts.normalised_dtype()
    model = load_model(model_dir, dtype, opts.device)
    engine = Engine(model, opts)
    ids = {}
    issued = 0
    for line in stream:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            if e["id"] not in ids:
                ids[e["id"]] = issued
                issued += 1
            entries.append(Entry(ids[e["id"]], [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])]))
        logits = engine.step(entries)
        if logits is not None:
            logits.detach().to(torch.float32).cpu().numpy().astype("<f4").tofile(os.path.join(out_dir, f"{step}.f32"))
        else:
            torch.cuda.synchronize()
        ops.raise_on_kernel_error()             # a kernel that gave up a bounded wait: no logits are better than wrong ones
        for name in rec.get("end", []):
            if name in ids:
                if engine.cache.is_live(ids[name]):
                    engine.release(ids[name])
                del ids[name]
        print(f"done {step}", flush=True)
    return 0
