#!/usr/bin/env python3
"""Benchmark of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl ours|reference]
    python bench.py --workload mix14b | 32b

Default run (the headline): decode tokens a second at batch 8, at batch 1 and 64, prefill of
2,048 tokens, and the same decode through the Python entry point with host tokens in and out.
Model: the sizes of Qwen3-8B (36 layers, width 4096, 32/8 heads of 128, feed-forward 12288,
vocabulary 151936), bfloat16, random weights; prompts are uniform random token ids.  A step is
one decode step of the whole batch at a context that ends at 4,096 tokens; the ids a step picks
are the next step's input (on the device), and the cache pages are handed out in a scattered
order, as after long serving.  `--layers` runs fewer layers of the same sizes (the record names
both numbers); layer sizes never shrink.

`--workload mix14b`: 32 requests with prompts of 128 to 2,048 tokens (seed-fixed) and 256 greedy
tokens each at the sizes of Qwen3-14B, through `LLM.add_request` / `LLM.step`, prompt portions
mixed with decode tokens under a budget of 512 tokens a step (two token tiles of the products).  `--workload 32b`: 16 requests of 1,024 + 128 tokens at
the sizes of Qwen3-32B (64 query heads of 128 on a width of 5,120).  Each prints one JSON line
with total, prompt and generated tokens a second, the time of all steps on the device, the
wall-clock time over it, and the steps' fraction of their roofline.

Timing: CUDA events on the launching stream around exactly K steps after W warm-up steps, with
a synchronize on both sides.  Every step streams all weights (15 GB) and the live requests'
cache from HBM, far more than the 126 MB of L2, so nothing a step reads is still cached from
the step before.  SM clocks and throttle reasons are sampled with nvidia-smi during the timed
regions.  One JSON line is printed.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=36, hidden_size=4096,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
                vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
                attention_bias=False, max_position_embeddings=40960, hidden_act="silu")
QWEN3_14B = dict(QWEN3_8B, num_hidden_layers=40, hidden_size=5120, num_attention_heads=40, intermediate_size=17408)
QWEN3_32B = dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, intermediate_size=25600)
# The reference cannot run this benchmark.  It is a CMake C11 project ("Neither 'setup.py' nor
# 'pyproject.toml' found" is pip's answer), its engine reads only its own quantized VQF files,
# and its one bfloat16-free route to the same numbers, the float32 CPU forward that
# tests/golden compiles, takes 35 ms a token and layer at these layer sizes on this machine's
# 8 cores (measured: 24 tokens through one layer, less 4 tokens through it, over 20) - 1.4 s a
# token for 36 layers and the output head - and prefills token by token
# (src/model/vllm_safetensors.c:17964-17971): the 8 x 2,048 prompt tokens of this benchmark
# alone would take more than six hours, and the float32 weights 33 GB of host memory.
REFERENCE_UNAVAILABLE = ("the reference is a CPU-only C11 engine (CMake, no Python package: pip install finds no setup.py or "
                         "pyproject.toml) that loads only its own quantized VQF files; its float32 forward, the one path "
                         "that takes these weights, was compiled and measured here at 35 ms per token and layer of this "
                         "size on 8 cores = 1.4 s a token, prefill token by token: batch 8 x context 4,096 would take hours")
CONTEXT = 4096
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                p = json.load(f)
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if isinstance(p.get(k), (int, float)) and p[k] > 0:
                    out[k] = float(p[k])
            out["source"] = "measured"
            return out
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 200 ms while `active`."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.rows = []
        self.active = False
        self._stop = False
        self._proc = None
        try:
            self._proc = subprocess.Popen(["nvidia-smi", f"--id={index}", f"--query-gpu={self.Q}",
                                           "--format=csv,noheader,nounits", "-lms", "200"],
                                          stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self._t = threading.Thread(target=self._read, daemon=True)
            self._t.start()
        except OSError:
            self._proc = None

    def _read(self):
        for line in self._proc.stdout:
            if self._stop:
                break
            if self.active:
                self.rows.append([c.strip() for c in line.split(",")])

    def close(self):
        self._stop = True
        if self._proc:
            self._proc.terminate()

    def summary(self):
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(int(float(r[0])))
                mx = max(mx, int(float(r[1])))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def run_workload(args) -> int:
    """A whole workload through the scheduler: requests are added to `LLM`, `LLM.step` is called
    until all are done; every step leaves CUDA events, from which the time on the device and the
    host's share follow."""
    import numpy as np
    import torch
    from kestrel_llm_b200 import LLM, SamplingParams
    from kestrel_llm_b200.config import EngineOptions, Qwen3Config
    from kestrel_llm_b200.config.registry import resolve_architecture
    from kestrel_llm_b200.weights import fill_random_

    if args.workload == "mix14b":
        raw, label = dict(QWEN3_14B), "Qwen3-14B shape"
        n_req, gen = args.requests or 32, args.generate or 256
        rng = np.random.default_rng(14)
        lengths = rng.integers(128, 2049, size=n_req).tolist()
        chunk = 512
        what = f"{n_req} requests, prompts of 128 to 2,048 tokens (seed 14), {gen} greedy tokens each, prompt portions of {chunk} mixed with decode tokens"
    else:
        raw, label = dict(QWEN3_32B), "Qwen3-32B shape"
        n_req, gen = args.requests or 16, args.generate or 128
        rng = np.random.default_rng(32)
        lengths = [1024] * n_req
        chunk = 512
        what = f"{n_req} requests of 1,024 prompt tokens, {gen} greedy tokens each, prompt portions of {chunk} mixed with decode tokens"
    full_layers = raw["num_hidden_layers"]
    if args.layers:
        raw["num_hidden_layers"] = min(args.layers, full_layers)
    cfg = Qwen3Config.from_dict(raw)
    L = cfg.num_hidden_layers
    dev = "cuda:0"
    torch.cuda.set_device(0)
    model = resolve_architecture(cfg.architecture).build(cfg, torch.bfloat16, dev)
    fill_random_(model, 0)
    longest = max(lengths) + gen + 64
    opts = EngineOptions(dtype="bfloat16", page_size=args.page_size, batch_max=n_req, max_model_len=longest,
                         max_tokens=sum(l + gen + 64 for l in lengths), max_step_tokens=max(args.step_tokens, chunk), prefill_batch=chunk)
    llm = LLM(model, dtype="bfloat16", options=opts)
    llm.engine.cache.shuffle_free(0)
    prompts = [rng.integers(0, cfg.vocab_size, size=n).tolist() for n in lengths]
    sp = SamplingParams(temperature=0.0, max_tokens=gen, ignore_eos=True)
    pk = peaks()
    # warm-up: a short run of the same kind, so that modules are loaded, graphs of the first buckets are captured and
    # the workspace has its size
    llm.generate([p[:300] for p in prompts[:min(4, n_req)]], SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    llm.warm_up()
    clocks = ClockSampler(0)
    llm.record_steps = True
    llm.step_records.clear()
    for p in prompts:
        llm.add_request(p, sp)
    contexts = []           # per step: (tokens, sum over entries of count * (start + (count + 1) / 2), live context tokens)
    sched_plan = llm.scheduler.schedule
    seen = []

    def watching():
        plan = sched_plan()
        seen.append(plan)
        return plan
    llm.scheduler.schedule = watching
    torch.cuda.synchronize()
    clocks.active = True
    t0 = time.perf_counter()
    done = llm.run_until_done()
    wall = time.perf_counter() - t0
    clocks.active = False
    clocks.close()
    llm.scheduler.schedule = sched_plan
    recs = llm.step_records
    dev_ms = [r.start.elapsed_time(r.end) for r in recs]
    device_s = sum(dev_ms) / 1000.0
    n_prompt, n_gen = sum(lengths), sum(len(o.token_ids) for o in done.values())
    # the steps' bound: every weight once, the live requests' cache, and the arithmetic, whichever is larger
    per_layer = (cfg.q_size + 2 * cfg.kv_size) * cfg.hidden_size + cfg.hidden_size * cfg.q_size + 3 * cfg.intermediate_size * cfg.hidden_size
    weight_bytes = 2 * (L * per_layer + cfg.vocab_size * cfg.hidden_size)
    kv_bytes_per_token = L * 2 * cfg.kv_size * 2
    plans = [p for p in seen if p]
    ideal_s, prefill_dev, decode_dev, mixed = 0.0, 0.0, 0.0, 0
    for plan, ms in zip(plans, dev_ms):
        T = sum(s.count for s in plan)
        ctx = sum(s.start + s.count for s in plan)
        pairs = sum(s.count * (s.start + (s.count + 1) / 2.0) for s in plan)
        flops = 2.0 * T * L * per_layer + 2.0 * sum(1 for s in plan if s.wants_token) * cfg.vocab_size * cfg.hidden_size \
            + L * 4.0 * cfg.num_attention_heads * cfg.head_dim * pairs
        byts = weight_bytes + ctx * kv_bytes_per_token
        ideal_s += max(byts / (pk["hbm_gbs"] * 1e9), flops / (pk["bf16_tflops_sustained"] * 1e12))
        if all(s.count == 1 for s in plan):
            decode_dev += ms
        else:
            prefill_dev += ms
            mixed += 1 if any(s.count == 1 for s in plan) else 0
    m = [o.metrics for o in done.values()]
    rec = {
        "metric": f"tokens/s (prompt + generated) of the workload, {label} bf16", "value": round((n_prompt + n_gen) / wall, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": len(recs), "warmup": 1, "ms_per_step": round(1000 * wall / max(1, len(recs)), 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights, uniform random token ids; " + what, "impl": "ours", "workload": args.workload,
        "config": {"model": label, "layers": L, "layers_of_model": full_layers, "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "requests": n_req, "generate": gen,
                   "prompt_tokens": n_prompt, "prefill_batch": chunk, "max_step_tokens": opts.max_step_tokens,
                   "page_size": args.page_size, "pages": "scattered", "parallelism": "single GPU", "peaks": pk["source"]},
        "wall_s": round(wall, 4), "device_s": round(device_s, 4), "wall_over_device": round(wall / device_s, 4),
        "prompt_tok_s": round(n_prompt / wall, 1), "generated_tok_s": round(n_gen / wall, 1),
        "steps_with_prompt_portions": {"steps": sum(1 for p in plans if any(s.count > 1 for s in p)), "of_them_mixed": mixed,
                                       "device_ms": round(prefill_dev, 2)},
        "decode_only_steps": {"steps": sum(1 for p in plans if all(s.count == 1 for s in p)), "device_ms": round(decode_dev, 2)},
        "roofline": {"bound": "per step max(bytes / HBM, flops / sustained bf16)", "ideal_s": round(ideal_s, 4),
                     "frac_of_device_time": round(ideal_s / device_s, 4), "frac_of_wall": round(ideal_s / wall, 4)},
        "requests": {"ttft_ms_mean": round(sum(x.ttft_ms for x in m) / len(m), 1), "ttft_ms_max": round(max(x.ttft_ms for x in m), 1),
                     "tpot_ms_mean": round(sum(x.tpot_ms for x in m) / len(m), 2), "preemptions": int(llm.scheduler.num_preemptions)},
        "gpu_launches": int(llm.engine.native_launches + llm.engine.graph_launches), "clocks": clocks.summary(),
    }
    print(json.dumps(rec))
    return 0


def main() -> int:
    global CONTEXT, PREFILL_TOKENS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--layers", type=int, default=0, help="run this many layers of the model's 36 (0 = all)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="leave out batch 1 and 64")
    ap.add_argument("--page-size", type=int, default=16, help="tokens per cache page (default 16)")
    ap.add_argument("--context", type=int, default=CONTEXT, help="context length at which the decode steps end (default 4096)")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS, help="tokens of the prefill step (default 2048)")
    ap.add_argument("--workload", default="decode8b", choices=["decode8b", "mix14b", "32b"],
                    help="decode8b: the headline run; mix14b / 32b: whole workloads through the scheduler")
    ap.add_argument("--requests", type=int, default=0, help="requests of a workload (0: 32 for mix14b, 16 for 32b)")
    ap.add_argument("--generate", type=int, default=0, help="tokens to generate per request of a workload (0: 256 / 128)")
    ap.add_argument("--step-tokens", type=int, default=2048,
                    help="token budget of a workload's step (the engine's default 2,048: up to four portions of 512 beside the decode tokens)")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on ONE GPU; --gpus {args.gpus} is not supported (no multi-GPU path exists)")
        return 2
    if args.workload != "decode8b":
        return run_workload(args)
    W, K = max(3, args.warmup), max(1, args.steps)
    CONTEXT, PREFILL_TOKENS = max(256, args.context), max(16, args.prefill_tokens)      # the defaults unless asked otherwise

    import numpy as np
    import torch
    from kestrel_llm_b200 import LLM, SamplingParams
    from kestrel_llm_b200.config import EngineOptions, Qwen3Config
    from kestrel_llm_b200.config.registry import resolve_architecture
    from kestrel_llm_b200.csrc import ops
    from kestrel_llm_b200.engine import Entry
    from kestrel_llm_b200.weights import fill_random_

    raw = dict(QWEN3_8B)
    full_layers = raw["num_hidden_layers"]
    if args.layers:
        raw["num_hidden_layers"] = min(args.layers, full_layers)
    cfg = Qwen3Config.from_dict(raw)
    L = cfg.num_hidden_layers
    dev = "cuda:0"
    torch.cuda.set_device(0)
    model = resolve_architecture(cfg.architecture).build(cfg, torch.bfloat16, dev)
    fill_random_(model, 0)
    max_batch = 64 if not args.skip_points else max(args.batch, 1)
    longest = max(CONTEXT, PREFILL_TOKENS) + 64
    opts = EngineOptions(dtype="bfloat16", page_size=args.page_size, batch_max=max_batch, max_model_len=longest,
                         max_tokens=max(max_batch * (CONTEXT + 64), longest), max_step_tokens=max(PREFILL_TOKENS, max_batch),
                         prefill_batch=PREFILL_TOKENS)
    llm = LLM(model, dtype="bfloat16", options=opts)
    engine = llm.engine
    engine.cache.shuffle_free(0)                     # pages in a scattered order, as after long serving
    for t in engine.cache.k + engine.cache.v:        # cache contents for the synthetic contexts
        if t is not None:
            t.normal_(0.0, 0.5)
    rng = np.random.default_rng(0)
    pk = peaks()
    clocks = ClockSampler(0)

    # bytes a decode step has to read: every weight it uses once, and the live requests' cache
    esz = 2
    per_layer = (cfg.q_size + 2 * cfg.kv_size) * cfg.hidden_size + cfg.hidden_size * cfg.q_size \
        + 3 * cfg.intermediate_size * cfg.hidden_size
    weight_bytes = esz * (L * per_layer + cfg.vocab_size * cfg.hidden_size)
    kv_bytes_per_token = L * 2 * cfg.kv_size * esz

    def timed(fn, n):
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        clocks.active = True
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        clocks.active = False
        return a.elapsed_time(b) / 1000.0

    def decode_point(B):
        """K timed decode steps of B requests whose context ends at CONTEXT; device-timed, the
        step function called directly, tokens picked on the device."""
        ctx0 = CONTEXT - (W + K)
        rids = list(range(1000, 1000 + B))
        for r in rids:
            engine.admit(r)
            engine.cache.reserve(r, ctx0)       # a context of ctx0 tokens whose cache holds random values
            engine.cache.commit(r, ctx0)
        nxt = torch.from_numpy(rng.integers(0, cfg.vocab_size, size=B).astype(np.int32)).to(dev)
        entries = [Entry(r, (0,), (0,)) for r in rids]       # the ids are on the device: those the step before picked

        def one():
            logits = engine.step(entries, token_ids_dev=nxt)
            ops.argmax(logits, nxt)

        for _ in range(W):
            one()
        before = ops.launches + engine.graph_launches + engine.native_launches
        secs = timed(one, K)
        launched = ops.launches + engine.graph_launches + engine.native_launches - before
        for r in rids:
            engine.release(r)
        mean_ctx = ctx0 + W + (K - 1) / 2.0 + 1
        bytes_step = weight_bytes + B * mean_ctx * kv_bytes_per_token
        return {"tok_s": B * K / secs, "ms": 1000.0 * secs / K, "bytes_step": bytes_step, "launches": launched}

    # prefill of one 2,048-token prompt in one step (logits of the last token); measured first: it
    # is bound by the tensor cores, whose clock sinks under the power cap once the GPU has been busy
    # for seconds, and its fraction is taken against the burst figure of the peak
    def prefill_once(rid):
        toks = rng.integers(0, cfg.vocab_size, size=PREFILL_TOKENS).tolist()
        engine.step([Entry(rid, toks, (PREFILL_TOKENS - 1,))])
        engine.release(rid)
    for i in range(2):
        prefill_once(2000 + i)
    pre_runs = 3
    counter = {"i": 0}

    def pf():
        counter["i"] += 1
        prefill_once(2100 + counter["i"])
    pre_secs = timed(pf, pre_runs) / pre_runs
    T = PREFILL_TOKENS
    gemm_flops = 2.0 * T * L * per_layer + 2.0 * cfg.vocab_size * cfg.hidden_size     # head: one row
    attn_flops = L * 4.0 * cfg.num_attention_heads * cfg.head_dim * (T * (T + 1) / 2.0)
    pre_flops = gemm_flops + attn_flops
    prefill = {"value": round(T / pre_secs, 1), "tokens": T, "ms": round(1000 * pre_secs, 3),
               "frac": round(pre_flops / pre_secs / (pk["bf16_tflops"] * 1e12), 4)}

    out_points = {}
    main_pt = decode_point(args.batch)
    if not args.skip_points:
        out_points["decode_b1"] = round(decode_point(1)["tok_s"], 2)
        out_points["decode_b64"] = round(decode_point(64)["tok_s"], 2)

    # end to end: the same decode through the Python entry point (scheduler, one H2D copy of the
    # step's description from pinned memory, sampling on the device, token ids read back)
    B = args.batch
    # while the prompts are still being prefilled (2,048 tokens a step) the first requests
    # already decode; every request must still be live when the timed steps end
    prefill_steps = -(-B * CONTEXT // opts.max_step_tokens)
    spare = prefill_steps + W + K + 8
    ctx0 = max(256, CONTEXT - spare)
    prompts = [rng.integers(0, cfg.vocab_size, size=ctx0).tolist() for _ in range(B)]
    sp = SamplingParams(temperature=0.0, max_tokens=spare + 32, ignore_eos=True)
    rids = [llm.add_request(p, sp) for p in prompts]
    while any(len(llm._live[r].out.token_ids) == 0 for r in rids):      # prompts, untimed
        llm.step()
    for _ in range(W):
        llm.step()
    h0, d0 = llm.stats.h2d_bytes, llm.stats.d2h_bytes
    torch.cuda.synchronize()
    clocks.active = True
    t0 = time.perf_counter()
    for _ in range(K):
        llm.step()                               # launches a step and reads back the ids of the one before
    torch.cuda.synchronize()
    e2e_secs = time.perf_counter() - t0
    clocks.active = False
    e2e = {"value": round(B * K / e2e_secs, 2), "unit": "tokens/s", "ms_per_step": round(1000 * e2e_secs / K, 3),
           "h2d_bytes_per_step": (llm.stats.h2d_bytes - h0) // K, "d2h_bytes_per_step": (llm.stats.d2h_bytes - d0) // K}
    for r in rids:
        llm.abort_request(r)
    clocks.close()

    achieved = main_pt["bytes_step"] / (main_pt["ms"] / 1000.0) / 1e9
    rec = {
        "metric": f"decode tokens/s, Qwen3-8B bf16, batch {args.batch}, context {CONTEXT}", "value": round(main_pt["tok_s"], 2),
        "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": round(main_pt["ms"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights, uniform random token ids, cache of the context filled with random values",
        "impl": "ours",
        "config": {"model": "Qwen3-8B shape", "layers": L, "layers_of_model": full_layers, "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "global_batch": args.batch,
                   "seq_len": CONTEXT, "page_size": args.page_size, "parallelism": "single GPU",
                   "cache_flush": "inputs larger than L2: each step streams all weights and cache from HBM",
                   "pages": "scattered", "token_feedback": "device",
                   "peaks": pk["source"]},
        "e2e": e2e, "gpu_launches": int(main_pt["launches"]), "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": out_points, "clocks": clocks.summary(),
    }
    print(json.dumps(rec))
    return 0


if __name__ == "__main__":
    sys.exit(main())
