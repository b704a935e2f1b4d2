"""Command line in the manner of the reference's ``src/main.c``: ``--flag value`` pairs,
one mode switch, tagged output lines.

Names and meanings taken over from the reference (src/main.c:4491-4850):
  --model DIR            model folder (main.c:4721)
  --stream-test          load, prefill the prompt, decode, print TOKIDS and timings (main.c:4725, 3140)
  --stream-n N           tokens to generate (main.c:4733)
  --stream-ctx N         pad the prompt to N tokens (main.c:4737)
  --warmup               one discarded prefill and 8 decode steps first (main.c:4727)
  --prefill-batch N      largest prompt portion of one step (main.c:4686)
  --batch-max N          live requests (main.c:4805)
  --max-queued N         waiting requests before admission refuses (main.c:4802)
  --top-k N, --min-p X   sampling filters (main.c:4567-4573)
  --repetition-penalty P, --repetition-window N   the harness's penalty on the last N generated
                         tokens (main.c:3741-3782; defaults from VLLM_STREAM_REPPEN / VLLM_STREAM_REPWIN)
Added for this engine: --plugin MODULE (imported first; it may register architectures of its
own), --profile, --debug-guards, --cuda-graphs 0|1, --dtype, --prompt-ids, --prompt-file, --random-prompts N:LEN:SEED,
--temperature, --top-p, --seed, --ignore-eos, --page-size, --max-tokens, --max-model-len,
--max-step-tokens, --random-weights SEED with --config FILE (writes the folder to --model
first), --replay (reads a trace on standard input, as bin/trace_run does, with --out DIR).
Output lines carry the reference's tags: ``[STREAM] prefill ...``, ``[STREAM] TOKIDS: ...``,
``[STREAM] decoded ...`` (main.c:3340, 3768, 3817).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time


def _repetition_options(args):
    """Penalty and window as the reference reads them (main.c:3741-3752): a penalty counts only
    if 1 < p < 1000, a window only if 1 <= n <= 64; otherwise off and 32."""
    pen, win = 1.0, 32
    raw = args.repetition_penalty if args.repetition_penalty is not None else os.environ.get("VLLM_STREAM_REPPEN", "")
    try:
        p = float(raw)
        if 1.0 < p < 1e3:
            pen = p
    except (TypeError, ValueError):
        pass
    raw = args.repetition_window if args.repetition_window is not None else os.environ.get("VLLM_STREAM_REPWIN", "")
    try:
        w = int(raw)
        if 1 <= w <= 64:
            win = w
    except (TypeError, ValueError):
        pass
    return pen, win


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="kestrel", description="Qwen3 dense decoder on one B200")
    ap.add_argument("--model", required=True)
    ap.add_argument("--stream-test", action="store_true")
    ap.add_argument("--stream-n", type=int, default=32)
    ap.add_argument("--stream-ctx", type=int, default=0)
    ap.add_argument("--warmup", action="store_true")
    ap.add_argument("--prefill-batch", type=int, default=512)
    ap.add_argument("--batch-max", type=int, default=32)
    ap.add_argument("--max-queued", type=int, default=16)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--min-p", type=float, default=0.0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--temperature", type=float, default=0.0)
    # the reference takes these two from the environment (main.c:3741-3752); the flags override it
    ap.add_argument("--repetition-penalty", type=float, default=None, help="default: VLLM_STREAM_REPPEN, else off")
    ap.add_argument("--repetition-window", type=int, default=None, help="default: VLLM_STREAM_REPWIN, else 32")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "bf16", "fp32"])
    ap.add_argument("--prompt-ids", default=None, help="comma-separated token ids")
    ap.add_argument("--prompt-file", default=None, help="one prompt a line, comma-separated token ids")
    ap.add_argument("--random-prompts", default=None, metavar="N:LEN:SEED")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--max-tokens", type=int, default=0, help="tokens the cache holds (0: batch-max * max-model-len)")
    ap.add_argument("--max-model-len", type=int, default=0)
    ap.add_argument("--max-step-tokens", type=int, default=2048)
    ap.add_argument("--random-weights", type=int, default=None, metavar="SEED")
    ap.add_argument("--config", default=None, help="config.json for --random-weights")
    ap.add_argument("--plugin", action="append", default=[], metavar="MODULE",
                    help="import this module first; it may register architectures and parts of its own (may be given several times)")
    ap.add_argument("--profile", action="store_true", help="time every step's phases on the device and print [DEC-SINGLE] / [PREFILL-TIMING] lines")
    ap.add_argument("--debug-guards", action="store_true", help="check every step's description on the device and guard words behind every activation")
    ap.add_argument("--cuda-graphs", type=int, default=1, help="0: launch decode steps kernel by kernel instead of replaying captured graphs")
    ap.add_argument("--replay", action="store_true")
    ap.add_argument("--out", default=None)
    return ap


def _prompts(args, vocab: int):
    import numpy as np
    if args.prompt_ids:
        return [[int(t) for t in args.prompt_ids.split(",") if t.strip()]]
    if args.prompt_file:
        with open(args.prompt_file) as f:
            return [[int(t) for t in line.split(",") if t.strip()] for line in f if line.strip()]
    if args.random_prompts:
        n, length, seed = (int(x) for x in args.random_prompts.split(":"))
        rng = np.random.default_rng(seed)
        return [rng.integers(0, vocab, size=length).tolist() for _ in range(n)]
    # the reference's harness uses a fixed chat prompt; without a tokenizer, a fixed id pattern
    return [[(7 * i + 3) % vocab for i in range(30)]]


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    import importlib
    for name in args.plugin:                  # architectures and parts from outside the package register themselves on import
        importlib.import_module(name)
    from . import LLM, SamplingParams
    from .config import EngineOptions, Qwen3Config, read_config_json, resolve_architecture, architecture_of
    from .weights import write_random_model

    if args.random_weights is not None:
        if not args.config:
            print("[STREAM] FAIL: --random-weights needs --config FILE", flush=True)
            return 2
        with open(args.config) as f:
            raw = json.load(f)
        cfg = resolve_architecture(architecture_of(raw)).config_class.from_dict(raw)
        write_random_model(cfg, args.random_weights, args.model, "bfloat16")
        print(f"[STREAM] random weights (seed {args.random_weights}) written to {args.model}", flush=True)
    if args.replay:
        from .engine.replay import replay_stdin
        return replay_stdin(args.model, args.dtype, args.out or "trace_out", args.max_tokens or 4096, args.page_size,
                            cuda_graphs=bool(args.cuda_graphs))

    t0 = time.perf_counter()
    llm = LLM(args.model, dtype=args.dtype, page_size=args.page_size, batch_max=args.batch_max,
              max_queued=max(args.max_queued, 1), prefill_batch=args.prefill_batch,
              max_step_tokens=args.max_step_tokens, max_tokens=args.max_tokens,
              max_model_len=args.max_model_len, seed=args.seed, profile=args.profile, debug_guards=args.debug_guards,
              cuda_graphs=bool(args.cuda_graphs))
    c = llm.model.config
    # sizes every architecture's configuration has; head counts where this one names them
    heads = "".join(f" {tag}={getattr(c, key)}" for tag, key in (("heads", "num_attention_heads"), ("kv", "num_key_value_heads"))
                    if hasattr(c, key))
    print(f"[STREAM] load OK ({time.perf_counter() - t0:.2f}s): arch={c.architecture} dim={c.hidden_size} "
          f"layers={c.num_hidden_layers}{heads} vocab={c.vocab_size} dtype={args.dtype}", flush=True)
    prompts = _prompts(args, c.vocab_size)
    if args.stream_ctx > 0:
        prompts = [(p * (args.stream_ctx // len(p) + 1))[:args.stream_ctx] for p in prompts]
    rep_pen, rep_win = _repetition_options(args)
    sp = SamplingParams(temperature=args.temperature, top_p=args.top_p, top_k=args.top_k, min_p=args.min_p,
                        max_tokens=args.stream_n, seed=args.seed, ignore_eos=args.ignore_eos,
                        repetition_penalty=rep_pen, repetition_window=rep_win)
    mode = "greedy" if sp.greedy else "sampling"
    print(f"[STREAM] decode mode: {mode}{'+reppen' if sp.penalised else ''} (rep_pen={rep_pen:.3f} win={rep_win})", flush=True)
    if args.warmup:
        tw = time.perf_counter()
        llm.generate(prompts[:1], SamplingParams(max_tokens=8, ignore_eos=True))
        print(f"[STREAM] warmup in {time.perf_counter() - tw:.3f}s (discarded: 1 prefill + 8 decode)", flush=True)
    import torch
    n_prompt = sum(len(p) for p in prompts)
    print(f"[STREAM] prompt tokens = {n_prompt} (--stream-ctx {args.stream_ctx}), requests = {len(prompts)}", flush=True)
    # prefill and decode are timed apart, as the reference's harness reports them
    for p in prompts:
        llm.add_request(p, sp)
    t1 = time.perf_counter()
    state = {"t_prefill": None}

    def after_step(finished):
        if state["t_prefill"] is None and llm.stats.generated_tokens >= len(prompts):
            torch.cuda.synchronize()
            state["t_prefill"] = time.perf_counter() - t1

    done = llm.run_until_done(after_step)         # raises if a kernel gave up a wait or nothing can run
    total = time.perf_counter() - t1
    t_prefill = state["t_prefill"]
    t_prefill = t_prefill if t_prefill is not None else total
    print(f"[STREAM] prefill {n_prompt} tokens in {t_prefill:.3f}s ({n_prompt / max(t_prefill, 1e-9):.0f} tok/s) [batch]", flush=True)
    mode = "greedy" if sp.greedy else f"sample T={sp.temperature} top_p={sp.top_p} top_k={sp.top_k} min_p={sp.min_p}"
    print(f"[STREAM] decode mode: {mode}", flush=True)
    for rid in sorted(done):
        print("[STREAM] TOKIDS: " + " ".join(str(t) for t in done[rid].token_ids), flush=True)
    n_dec = sum(len(o.token_ids) for o in done.values()) - len(prompts)
    t_dec = max(total - t_prefill, 1e-9)
    if n_dec > 0:
        print(f"[STREAM] decoded {n_dec} tokens, {1000 * t_dec / n_dec:.2f} ms/tok ({n_dec / t_dec:.2f} tok/s)", flush=True)
    for rid in sorted(done):
        m = done[rid].metrics
        print(f"[STREAM] metrics request={rid} prompt_tokens={m.prompt_tokens} n_tokens={m.n_tokens} prefill_ms={m.prefill_ms:.1f} "
              f"ttft_ms={m.ttft_ms:.1f} tpot_ms={m.tpot_ms:.2f} total_ms={m.total_ms:.1f} finish={done[rid].finish_reason}", flush=True)
    occ = llm.cache_occupancy()
    for i, g in enumerate(occ["groups"]):
        print(f"[STREAM] cache group {i}: window={g['window']} pages={g['pages']} free={g['free']} page_size={occ['page_size']} "
              f"preemptions={llm.scheduler.num_preemptions}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
