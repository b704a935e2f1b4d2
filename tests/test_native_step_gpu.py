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
