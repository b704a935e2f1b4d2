"""The two ways a step's kernels get launched - the native runner walking the model's step
program, and the parts' forward methods called from Python - run the same kernels in the same
order on the same inputs, so their logits must be the same bits, in float32 and in bfloat16;
and the Python walk, which models with parts of their own fall back to, is held against the
plain implementation by itself (GPU)."""
import numpy as np
import pytest

import replay_util as R
import tiny_configs
from test_replay_gpu import LENGTHS, LENGTHS_MIXED, _requests

pytestmark = pytest.mark.gpu

DTYPES = ("float32", "bfloat16")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
def test_native_runner_and_python_walk_give_the_same_bits(model_dirs, name, dtype):
    reqs = _requests(name, LENGTHS_MIXED.get(name))
    for family in (R.trace_mixed, R.trace_portions):
        steps, max_tokens = family(reqs)
        native = R.make_engine(model_dirs[name][dtype], dtype, max_tokens, native=True)
        walked = R.make_engine(model_dirs[name][dtype], dtype, max_tokens, native=False)
        assert native.runner is not None and walked.runner is None
        a = R.run_trace(native, steps)
        b = R.run_trace(walked, steps)
        assert native.native_launches > 0 and walked.native_launches == 0
        for rname, toks in reqs.items():
            for p in range(len(toks)):
                assert np.array_equal(a[rname][p], b[rname][p]), \
                    f"{family.__name__}: request {rname} position {p}: the two walks differ by " \
                    f"{np.abs(a[rname][p] - b[rname][p]).max():.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "D"])
@pytest.mark.parametrize("family", [R.trace_whole, R.trace_tail_decode, R.trace_portions, R.trace_mixed])
def test_python_walk_against_the_plain_implementation(model_dirs, name, dtype, family):
    reqs = _requests(name, LENGTHS_MIXED[name] if family is R.trace_mixed else None)
    steps, max_tokens = family(reqs)
    engine = R.make_engine(model_dirs[name][dtype], dtype, max_tokens, native=False)
    got = R.run_trace(engine, steps)
    R.compare_with_plain(model_dirs[name]["float32"], reqs, got, dtype, f"walk/{name}/{dtype}/{family.__name__}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "D"])
def test_debug_guards_stay_quiet_on_valid_steps(model_dirs, name, dtype):
    """With the debug guards on, every step's description is checked on the device before a
    kernel indexes with it, and guard words behind every activation are read back: on valid
    steps nothing is reported and the logits are those of the unguarded engine."""
    reqs = _requests(name, LENGTHS_MIXED[name])
    steps, max_tokens = R.trace_mixed(reqs)
    guarded = R.make_engine(model_dirs[name][dtype], dtype, max_tokens, guards=True)
    plain = R.make_engine(model_dirs[name][dtype], dtype, max_tokens)
    a = R.run_trace(guarded, steps)
    b = R.run_trace(plain, steps)
    assert guarded.runner.guard_failures == 0
    for rname, toks in reqs.items():
        for p in range(len(toks)):
            assert np.array_equal(a[rname][p], b[rname][p])


def test_profile_prints_the_reference_lines(model_dirs, capsys):
    """`EngineOptions.profile`: every step's phases are timed on the device and printed in the
    reference's formats - `[PREFILL-TIMING]` / `[PREFILL-KERNELS]` for steps with prompt portions,
    `[DEC-SINGLE]` for steps of single tokens - and the tokens are those of the unprofiled run."""
    import re
    from kestrel_llm_b200 import LLM, SamplingParams
    prompts = list(R.random_requests(509, (40, 9), seed=3).values())
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    plain = LLM(model_dirs["B"]["bfloat16"], dtype="bfloat16", max_tokens=512, batch_max=2).generate(prompts, sp)
    capsys.readouterr()
    llm = LLM(model_dirs["B"]["bfloat16"], dtype="bfloat16", max_tokens=512, batch_max=2, profile=True)
    outs = llm.generate(prompts, sp)
    err = capsys.readouterr().err
    assert [o.token_ids for o in outs] == [o.token_ids for o in plain]
    pre = re.findall(r"\[PREFILL-TIMING\] n=(\d+) total=([0-9.]+)ms \| GEMM=([0-9.]+)ms\(.*?\) ATTN=([0-9.]+)ms\(.*?\) OTHER=([0-9.]+)ms", err)
    assert pre and int(pre[0][0]) == 49 and float(pre[0][1]) > 0 and float(pre[0][2]) > 0
    from kestrel_llm_b200.csrc import ops
    prof = llm.engine.profile            # the line prints tenths of a millisecond; the sums behind it are finer
    assert all(prof.prefill_ms[ops.PHASES[k]] > 0 for k in ("qkv", "attn", "o", "gate_up", "down", "norm", "rope", "lm_head", "embed"))
    assert "[PREFILL-KERNELS] QKV=" in err
    dec = re.findall(r"\[DEC-SINGLE\] seq=(\d+) qkv=([0-9.]+) attn=([0-9.]+) o=([0-9.]+) gu=([0-9.]+) down=([0-9.]+) lm=([0-9.]+) nrm=([0-9.]+) rope=([0-9.]+)", err)
    assert len(dec) == 5 and all(prof.decode_ms[ops.PHASES[k]] > 0 for k in ("qkv", "attn", "o", "gate_up", "down", "norm", "rope", "lm_head"))
    assert llm.engine.profile.decode_steps == 5 and llm.engine.profile.prefill_steps == 1


def test_request_metrics_and_cache_occupancy(model_dirs):
    """Every finished request carries the reference's six numbers (VLLMMetrics), and the pool's
    occupancy can be read while requests are live."""
    from kestrel_llm_b200 import LLM, SamplingParams
    llm = LLM(model_dirs["B"]["bfloat16"], dtype="bfloat16", max_tokens=512, batch_max=4, page_size=16)
    prompts = list(R.random_requests(509, (30, 5, 64), seed=9).values())
    rids = [llm.add_request(p, SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=True)) for p, n in zip(prompts, (7, 1, 12))]
    first = {o.request_id: o for o in llm.step()}          # the request that wants one token is over after the first step
    occ = llm.cache_occupancy()
    assert list(first) == [rids[1]] and occ["live_requests"] == 2 and occ["running"] == 2 and occ["waiting"] == 0
    assert occ["groups"][0]["free"] < occ["groups"][0]["pages"] and occ["page_size"] == 16
    done = {**first, **llm.run_until_done()}
    for rid, p, n in zip(rids, prompts, (7, 1, 12)):
        m = done[rid].metrics
        assert m.prompt_tokens == len(p) and m.n_tokens == n == len(done[rid].token_ids)
        assert 0 < m.prefill_ms <= m.ttft_ms <= m.total_ms
        assert (m.tpot_ms == m.ttft_ms) if n == 1 else abs(m.tpot_ms * (n - 1) - (m.total_ms - m.ttft_ms)) < 1e-6
    occ = llm.cache_occupancy()
    assert occ["live_requests"] == 0 and occ["groups"][0]["free"] == occ["groups"][0]["pages"]
