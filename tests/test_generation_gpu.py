"""Generation through the Python entry point, long decoding, the first tokens of a sequence,
what happens when pages run out, and the command line (GPU)."""
import os
import subprocess
import sys

import numpy as np
import pytest

import plain_qwen3 as P
import replay_util as R
import tiny_configs

pytestmark = pytest.mark.gpu


def _check_greedy(model_dir_f32, prompt, generated, dtype):
    cfg, W = P.read_model(model_dir_f32)
    toks = list(prompt)
    for got in generated:
        logits = P.forward_logits(cfg, W, toks)[-1]
        want = P.greedy(logits)
        if got != want:     # only a tie within rounding may differ
            assert float(logits[want] - logits[got]) <= R.TOL[dtype] * float(np.abs(logits).max()), \
                f"token {got} instead of {want} after {len(toks)} tokens"
        toks.append(got)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,lengths,n_new,chunk", [("A", (5, 11, 17), 8, 512), ("B", (1, 33, 70, 129), 16, 24)])
def test_greedy_generation(model_dirs, name, lengths, n_new, chunk, dtype):
    """The workloads of the two tiny baseline configurations, greedy, through LLM.generate."""
    from kestrel_llm_b200 import LLM, SamplingParams
    prompts = list(R.random_requests(tiny_configs.CONFIGS[name][0]["vocab_size"], lengths, seed=1 if name == "A" else 3).values())
    page = 4 if name == "A" else 16
    llm = LLM(model_dirs[name][dtype], dtype=dtype, page_size=page, batch_max=4, max_tokens=1024,
              prefill_batch=chunk, max_step_tokens=64)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=n_new, ignore_eos=True))
    assert [len(o.token_ids) for o in outs] == [n_new] * len(prompts)
    assert all(o.finish_reason == "length" for o in outs)
    for p, o in zip(prompts, outs):
        _check_greedy(model_dirs[name]["float32"], p, o.token_ids, dtype)
    assert llm.engine.cache.live_requests() == 0
    llm.engine.cache.check()
    assert llm.stats.generated_tokens == n_new * len(prompts) and llm.stats.d2h_bytes == 4 * llm.stats.generated_tokens
    # twice the same: token ids are stable from run to run
    again = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=n_new, ignore_eos=True))
    assert [o.token_ids for o in again] == [o.token_ids for o in outs]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_with_a_repetition_penalty(model_dirs, dtype):
    """The harness's repetition penalty on the last generated tokens, greedy, beside a request
    without one (which still runs ahead of the host when it is alone): every token is the first
    maximum of the plain implementation's penalised logits."""
    from kestrel_llm_b200 import LLM, SamplingParams
    prompts = list(R.random_requests(tiny_configs.A["vocab_size"], (9, 21), seed=6).values())
    llm = LLM(model_dirs["A"][dtype], dtype=dtype, page_size=16, batch_max=4, max_tokens=1024)
    sps = [SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True, repetition_penalty=1.8, repetition_window=6),
           SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True)]
    outs = llm.generate(prompts, sps)
    cfg, W = P.read_model(model_dirs["A"]["float32"])
    toks, gen = list(prompts[0]), []
    for got in outs[0].token_ids:
        logits = P.repetition_penalty(P.forward_logits(cfg, W, toks)[-1], gen, 1.8, 6)
        want = P.greedy(logits)
        if got != want:
            assert float(logits[want] - logits[got]) <= R.TOL[dtype] * float(np.abs(logits).max()), \
                f"token {got} instead of {want} after {len(gen)} generated tokens"
        toks.append(got)
        gen.append(got)
    _check_greedy(model_dirs["A"]["float32"], prompts[1], outs[1].token_ids, dtype)
    plain = llm.generate(prompts[:1], SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True))[0].token_ids
    assert plain != outs[0].token_ids, "the penalty changed nothing: the test shows nothing"
    with pytest.raises(ValueError, match="repetition_window"):
        SamplingParams(repetition_window=65)


def test_temperature_sampling_does_not_depend_on_the_batch(model_dirs):
    """Config B's workload: temperature 0.8, seed 4, 16 tokens, portions of 24 beside decodes.
    A request's tokens are the same alone and in company, and follow the plain sampler fed with
    the plain logits and the same uniform numbers."""
    from kestrel_llm_b200 import LLM, SamplingParams
    from kestrel_llm_b200.sampling import uniform_for
    prompts = list(R.random_requests(509, (1, 33, 70, 129), seed=3).values())
    sp = [SamplingParams(temperature=0.8, max_tokens=16, seed=4 + i, ignore_eos=True) for i in range(4)]
    together = LLM(model_dirs["B"]["float32"], dtype="float32", page_size=16, batch_max=4, max_tokens=1024,
                   prefill_batch=24, max_step_tokens=48).generate(prompts, sp)
    alone = [LLM(model_dirs["B"]["float32"], dtype="float32", page_size=16, batch_max=1, max_tokens=256)
             .generate([p], s)[0] for p, s in zip(prompts, sp)]
    assert [o.token_ids for o in together] == [o.token_ids for o in alone]
    cfg, W = P.read_model(model_dirs["B"]["float32"])
    for i in (0, 2):
        toks = list(prompts[i])
        for j, got in enumerate(together[i].token_ids):
            p = P.sample_probs(P.forward_logits(cfg, W, toks)[-1], 0.8)
            want = P.sample_from(p, uniform_for(4 + i, j))
            if got != want:
                c = np.cumsum(p.astype(np.float64))
                assert abs(c[min(got, want)] - uniform_for(4 + i, j) * c[-1]) < 1e-4 * c[-1]
            toks.append(got)
    other = LLM(model_dirs["B"]["float32"], dtype="float32", max_tokens=256, batch_max=1).generate(
        [prompts[1]], SamplingParams(temperature=0.8, max_tokens=16, seed=99, ignore_eos=True))[0]
    assert other.token_ids != together[1].token_ids


def test_decoding_far_into_a_long_context(tmp_path):
    """17,000 tokens of context, head size 128: the captured decode step of that context class
    cuts the key range into more slices than a cluster merges (scratch and a merge kernel inside
    the graph), and a second, short request decodes beside it.  The logits agree with the
    uncaptured engine's (which picks its slices per step) within bfloat16 rounding, and with
    themselves from one class of context to the next."""
    import torch
    from kestrel_llm_b200.config import Qwen3Config
    from kestrel_llm_b200.weights import write_random_model
    raw = dict(tiny_configs.D, max_position_embeddings=20000, num_hidden_layers=2)
    raw.pop("sliding_window"); raw.pop("use_sliding_window"); raw.pop("layer_types")
    model_dir = str(tmp_path / "long")
    write_random_model(Qwen3Config.from_dict(raw), 3, model_dir, "bfloat16")
    rng = np.random.default_rng(4)
    long_req = rng.integers(0, raw["vocab_size"], size=17003).tolist()
    short_req = rng.integers(0, raw["vocab_size"], size=40).tolist()
    steps = []
    n, chunk = 0, 2048
    while n < 17000:
        k = min(chunk, 17000 - n)
        steps.append({"entries": [{"id": "long", "tokens": long_req[n:n + k], "want": []}], "end": []})
        n += k
    steps.append({"entries": [{"id": "short", "tokens": short_req[:37], "want": []}], "end": []})
    for i in range(3):
        steps.append({"entries": [{"id": "long", "tokens": [long_req[17000 + i]], "want": [0]},
                                  {"id": "short", "tokens": [short_req[37 + i]], "want": [0]}], "end": []})
    steps[-1]["end"] = ["long", "short"]
    results = []
    for graphs in (False, True):
        engine = R.make_engine(model_dir, "bfloat16", 17003 + 64 + 128, graphs=graphs)
        results.append(R.run_trace(engine, steps))
        if graphs:
            assert engine.graph_launches > 0
            assert any(k[1] > 16384 for k in engine.graphs._graphs), "the long context has a class of its own"
        torch.cuda.synchronize()
    for name in ("long", "short"):
        for pos, row in results[0][name].items():
            other = results[1][name][pos]
            assert np.isfinite(row).all() and np.isfinite(other).all()
            err = float(np.abs(row - other).max()) / float(np.abs(row).max())
            assert err <= R.TOL["bfloat16"], f"{name} position {pos}: captured and uncaptured steps differ by {err:.3e}"


def test_stop_token_ends_a_request(model_dirs):
    from kestrel_llm_b200 import LLM, SamplingParams
    prompt = R.random_requests(256, (9,), seed=5)["r0"]
    llm = LLM(model_dirs["A"]["float32"], dtype="float32", max_tokens=256, batch_max=2)
    free = llm.generate([prompt], SamplingParams(max_tokens=8, ignore_eos=True))[0].token_ids
    stop = free[3]
    cut = llm.generate([prompt], SamplingParams(max_tokens=8, stop_token_ids=(stop,)))[0]
    k = free.index(stop)
    assert cut.finish_reason == "stop" and cut.token_ids == free[:k + 1]


def test_decode_steps_that_run_ahead_change_no_token(model_dirs):
    """bfloat16 with captured decode steps: the next step is launched before the host has read
    the last one's ids.  Requests that stop at different times (a stop token found one step late,
    different token limits, one request joining later) give the same ids as with every step read
    back at once, nothing is left in the cache, and a stopped request's extra token is dropped."""
    from kestrel_llm_b200 import LLM, SamplingParams
    prompts = list(R.random_requests(509, (7, 40, 3, 90), seed=11).values())

    def run(run_ahead, params, late=None):
        llm = LLM(model_dirs["B"]["bfloat16"], dtype="bfloat16", page_size=16, batch_max=4, max_tokens=2048,
                  prefill_batch=64, max_step_tokens=128)
        llm.run_ahead = run_ahead
        rids = [llm.add_request(p, sp) for p, sp in zip(prompts, params)]
        done, steps = {}, 0
        while llm.has_unfinished():
            for o in llm.step():
                done[o.request_id] = o
            steps += 1
            if late is not None and steps == 12:            # a request arrives while the others decode
                rids.append(llm.add_request(late[0], late[1]))
        assert llm.engine.cache.live_requests() == 0
        llm.engine.cache.check()
        return [done[r] for r in rids], llm

    free = [SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=True) for n in (40, 25, 33, 40)]
    base, _ = run(False, free)
    ahead, llm = run(True, free)
    assert [o.token_ids for o in ahead] == [o.token_ids for o in base]
    assert [len(o.token_ids) for o in ahead] == [40, 25, 33, 40]
    assert llm.stats.generated_tokens == 138
    # stop tokens taken from the free run, at different depths; temperature sampling for one request
    stops = [SamplingParams(temperature=0.0, max_tokens=40, stop_token_ids=(base[0].token_ids[17],)),
             SamplingParams(temperature=0.0, max_tokens=25, ignore_eos=True),
             SamplingParams(temperature=0.9, top_k=20, seed=5, max_tokens=33, ignore_eos=True),
             SamplingParams(temperature=0.0, max_tokens=40, stop_token_ids=(base[3].token_ids[5], base[3].token_ids[30]))]
    late = (prompts[1][:20], SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    b2, _ = run(False, stops, late)
    a2, llm2 = run(True, stops, late)
    assert [o.token_ids for o in a2] == [o.token_ids for o in b2]
    assert [o.finish_reason for o in a2] == [o.finish_reason for o in b2]
    assert a2[0].finish_reason == "stop" and a2[3].finish_reason == "stop" and a2[1].finish_reason == "length"
    assert a2[0].token_ids[-1] == base[0].token_ids[17] and len(a2[0].token_ids) <= 18
    # ids thrown away were still copied: more bytes read back than tokens kept
    assert llm2.stats.d2h_bytes >= 4 * llm2.stats.generated_tokens


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(model_dirs, dtype, record_property):
    """Four prompt tokens, then 300 tokens one by one: every position against the plain
    implementation, across many page edges."""
    reqs = R.random_requests(509, (304,), seed=8)
    steps, max_tokens = R.trace_tail_decode(reqs, tail=300)
    assert len(steps) == 301
    got = R.run_trace(R.make_engine(model_dirs["B"][dtype], dtype, max_tokens), steps)
    R.compare_with_plain(model_dirs["B"]["float32"], reqs, got, dtype, "long decode")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_first_tokens_of_a_sequence(model_dirs, name, dtype):
    vocab = tiny_configs.CONFIGS[name][0]["vocab_size"]
    reqs = R.random_requests(vocab, (1, 2, 3, 4), seed=6)
    for family in (R.trace_whole, R.trace_tail_decode):
        steps, max_tokens = family(reqs)
        got = R.run_trace(R.make_engine(model_dirs[name][dtype], dtype, max_tokens, page_size=4), steps)
        R.compare_with_plain(model_dirs[name]["float32"], reqs, got, dtype, f"first tokens {family.__name__}")


@pytest.mark.parametrize("sampling", ["greedy", "temperature", "penalty"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_when_pages_run_out_the_youngest_is_computed_again(model_dirs, dtype, sampling):
    """A pool too small for all requests at their full length: requests are preempted and
    recomputed, and still produce the tokens they produce undisturbed - with greedy picking, with
    seeded temperature sampling (the uniform number of a request's token j is a function of its
    seed and j, so it is the same after recomputation) and with a repetition penalty (which
    needs the generated tokens on the host).  In bfloat16 decode steps are captured and run ahead
    of the host while no one waits.

    The recomputation runs a request's generated tokens as part of a prompt portion, by other
    kernels than the decode steps that first computed them; in float32 that changes no bit, in
    bfloat16 it may flip a token whose two best logits are within rounding of each other, so the
    bfloat16 runs are compared through the plain implementation's margin at the first difference."""
    from kestrel_llm_b200 import LLM, SamplingParams
    prompts = list(R.random_requests(509, (30, 28, 33), seed=12).values())
    if sampling == "greedy":
        sps = [SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True)] * 3
    elif sampling == "temperature":
        sps = [SamplingParams(temperature=0.8, top_k=40, seed=100 + i, max_tokens=40, ignore_eos=True) for i in range(3)]
    else:
        sps = [SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True, repetition_penalty=1.3, repetition_window=16)] * 3
    roomy_llm = LLM(model_dirs["B"][dtype], dtype=dtype, page_size=16, batch_max=4, max_tokens=1024)
    roomy = roomy_llm.generate(prompts, sps)
    tight_llm = LLM(model_dirs["B"][dtype], dtype=dtype, page_size=16, batch_max=4, num_pages=9)   # 144 tokens
    tight = tight_llm.generate(prompts, sps)
    assert tight_llm.scheduler.num_preemptions > 0 and sum(o.preemptions for o in tight) > 0
    if dtype == "bfloat16":
        assert tight_llm.engine.graph_launches > 0          # decode steps were replayed from graphs
    for o_t, o_r, prompt in zip(tight, roomy, prompts):
        if o_t.token_ids == o_r.token_ids:
            continue
        assert dtype == "bfloat16", "float32 logits do not depend on the cutting: the tokens must be the same"
        # first difference: both tokens must be near-ties for the plain implementation
        k = next(i for i, (x, y) in enumerate(zip(o_t.token_ids, o_r.token_ids)) if x != y)
        cfg, W = P.read_model(model_dirs["B"]["float32"])
        row = P.forward_logits(cfg, W, list(prompt) + o_r.token_ids[:k])[-1]
        if sampling == "penalty":
            row = P.repetition_penalty(row, o_r.token_ids[:k], 1.3, 16)
        gap = abs(float(row[o_t.token_ids[k]]) - float(row[o_r.token_ids[k]]))
        if sampling == "temperature":
            p = P.sample_probs(row, 0.8, top_k=40)
            c = np.cumsum(p.astype(np.float64)) / float(p.sum())
            lo, hi = sorted((o_t.token_ids[k], o_r.token_ids[k]))
            assert hi - lo <= 2 or abs(c[lo] - c[hi - 1]) < 2e-2, f"token {k}: {o_t.token_ids[k]} against {o_r.token_ids[k]}"
        else:
            assert gap <= 2e-2 * float(np.abs(row).max()), f"token {k} differs with a margin of {gap:.3e}"
    tight_llm.engine.cache.check()
    assert tight_llm.engine.cache.live_requests() == 0


def test_requests_that_cannot_run_are_refused(model_dirs):
    from kestrel_llm_b200 import LLM, SamplingParams
    from kestrel_llm_b200.engine import SchedulerError
    llm = LLM(model_dirs["A"]["float32"], dtype="float32", num_pages=4, page_size=16, batch_max=2)
    with pytest.raises(SchedulerError, match="exceed"):
        llm.add_request(list(range(60)), SamplingParams(max_tokens=10))
    with pytest.raises(ValueError, match="outside the vocabulary"):
        llm.add_request([1, 2, 256])
    from kestrel_llm_b200.engine import Entry
    with pytest.raises(ValueError, match="outside the vocabulary"):
        llm.engine.step([Entry(0, [999], [0])])
    with pytest.raises(ValueError, match="outside its"):
        llm.engine.step([Entry(0, [1, 2], [2])])
    assert llm.engine.cache.live_requests() == 0


def test_command_line(model_dirs):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "kestrel"), "--model", model_dirs["A"]["bfloat16"],
                        "--stream-test", "--stream-n", "6", "--prompt-ids", "5,17,3,200", "--dtype", "float32"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    line = [l for l in p.stdout.splitlines() if l.startswith("[STREAM] TOKIDS:")]
    assert len(line) == 1
    ids = [int(t) for t in line[0].split(":", 1)[1].split()]
    assert len(ids) == 6
    _check_greedy(model_dirs["A"]["float32"], [5, 17, 3, 200], ids, "float32")
    assert "[STREAM] decode mode: greedy (rep_pen=1.000 win=32)" in p.stdout
    # the reference's environment variable switches the repetition penalty on, a flag overrides the window
    env = dict(os.environ, VLLM_STREAM_REPPEN="1.7")
    q = subprocess.run([sys.executable, os.path.join(root, "bin", "kestrel"), "--model", model_dirs["A"]["bfloat16"],
                        "--stream-test", "--stream-n", "12", "--prompt-ids", "5,17,3,200", "--dtype", "float32",
                        "--repetition-window", "5"], capture_output=True, text=True, timeout=600, env=env)
    assert q.returncode == 0, q.stderr[-2000:]
    assert "[STREAM] decode mode: greedy+reppen (rep_pen=1.700 win=5)" in q.stdout
    line = [l for l in q.stdout.splitlines() if l.startswith("[STREAM] TOKIDS:")]
    got = [int(t) for t in line[0].split(":", 1)[1].split()]
    cfg, W = P.read_model(model_dirs["A"]["float32"])
    toks, gen = [5, 17, 3, 200], []
    for g in got:
        logits = P.repetition_penalty(P.forward_logits(cfg, W, toks)[-1], gen, 1.7, 5)
        want = P.greedy(logits)
        assert g == want or float(logits[want] - logits[g]) <= R.TOL["float32"] * float(np.abs(logits).max())
        toks.append(g)
        gen.append(g)
