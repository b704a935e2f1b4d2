"""The engine against the plain implementation under every way of cutting the work, in
float32 and in bfloat16, for five tiny configurations (GPU)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import replay_util as R
import tiny_configs

pytestmark = pytest.mark.gpu

LENGTHS = {"A": (5, 11, 17, 40, 70), "B": (1, 33, 70, 129, 47, 90), "C": (3, 50, 97, 130, 64, 81),
           "D": (2, 45, 131, 200, 77), "E": (9, 64, 150, 129), "F": (4, 40, 150, 66)}
# more requests than fit the pool at once, so that finished requests' pages are used again
LENGTHS_MIXED = {"A": (5, 11, 17, 40, 70, 64, 33, 90, 25, 70, 48), "B": (1, 33, 70, 129, 47, 90, 16, 65, 120, 31),
                 "C": (3, 50, 97, 130, 64, 81, 17, 111, 49, 128), "D": (2, 45, 131, 200, 77, 33, 160, 90, 64),
                 "E": (9, 64, 150, 129, 40, 100, 65, 31)}
DTYPES = ("float32", "bfloat16")


def _requests(name, lengths=None):
    return R.random_requests(tiny_configs.CONFIGS[name][0]["vocab_size"], lengths or LENGTHS[name], seed=1 + ord(name))


def _run(model_dirs, name, dtype, family, record_property, lengths=None, graphs=False, page_size=16, **kw):
    reqs = _requests(name, lengths)
    steps, max_tokens = family(reqs, **kw)
    engine = R.make_engine(model_dirs[name][dtype], dtype, max_tokens, graphs=graphs, page_size=page_size)
    got = R.run_trace(engine, steps)
    assert engine.cache.live_requests() == 0
    engine.cache.check()
    worst = R.compare_with_plain(model_dirs[name]["float32"], reqs, got, dtype, f"{name}/{dtype}/{family.__name__}")
    record_property("worst_relative_error", worst)
    print(f"[replay] {name} {dtype} {family.__name__}: worst {worst:.3e}")
    return engine


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_whole_prompts(model_dirs, name, dtype, record_property):
    _run(model_dirs, name, dtype, R.trace_whole, record_property)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("family", [R.trace_whole, R.trace_tail_decode])
def test_more_heads_per_kv_head_than_a_decode_tile_holds(model_dirs, dtype, family, record_property):
    """18 query heads on one kv head: a token's rows do not fit the 16-row tiles, so decode
    tokens run on the kernels for prompt portions and the model's steps are not captured."""
    engine = _run(model_dirs, "F", dtype, family, record_property, graphs=True)
    assert engine.graphs is None and engine.graph_launches == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_last_tokens_one_by_one(model_dirs, name, dtype, record_property):
    _run(model_dirs, name, dtype, R.trace_tail_decode, record_property)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
@pytest.mark.parametrize("family", ["tail", "mixed"])
def test_decode_steps_replayed_from_cuda_graphs(model_dirs, name, dtype, family, record_property):
    """The same traces with decode-only steps captured once per batch-size bucket and replayed
    (what generation does); prompt portions and mixed steps still launch kernel by kernel."""
    if family == "tail":
        engine = _run(model_dirs, name, dtype, R.trace_tail_decode, record_property, graphs=True)
    else:
        engine = _run(model_dirs, name, dtype, R.trace_mixed, record_property, lengths=LENGTHS_MIXED[name], graphs=True,
                      tail=24)
    assert engine.graphs is not None and engine.graph_launches > 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_portions_of_changing_size(model_dirs, name, dtype, record_property):
    _run(model_dirs, name, dtype, R.trace_portions, record_property)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_mixed_with_page_reuse(model_dirs, name, dtype, record_property):
    engine = _run(model_dirs, name, dtype, R.trace_mixed, record_property, lengths=LENGTHS_MIXED[name])
    # the pool was so small that pages were handed out more often than there are pages
    assert engine.cache.pages_handed_out() > engine.cache.num_pages(0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,page_size", [("A", 4), ("D", 8), ("D", 32), ("E", 64), ("B", 8)])
@pytest.mark.parametrize("family", [R.trace_whole, R.trace_tail_decode, R.trace_portions, R.trace_mixed])
def test_other_page_sizes(model_dirs, name, page_size, family, dtype, record_property):
    """The four families again with other pages than 16 tokens: 4 (the first baseline
    configuration's; in bfloat16 such pages take the mma.sync kernels for portions and for
    decode tokens), 8 and 32 at head size 128 (several pages to a key tile of the TMA-fed
    kernels, and a page of two decode tiles), 64 at head size 64."""
    lengths = LENGTHS_MIXED[name] if family is R.trace_mixed else None
    engine = _run(model_dirs, name, dtype, family, record_property, lengths=lengths, page_size=page_size,
                  graphs=(family is R.trace_tail_decode))
    if family is R.trace_mixed:
        assert engine.cache.pages_handed_out() > engine.cache.num_pages(0)


@pytest.mark.parametrize("per_cent", [0, 100, 1000])
@pytest.mark.parametrize("family", [R.trace_portions, R.trace_mixed])
def test_short_portions_on_either_attention_kernel(model_dirs, per_cent, family, record_property):
    """Head size 128 in bfloat16: short portions go to the attention kernel for decode tokens
    while their keys are few (the default), never (0), or whatever their keys (1000); every
    route against the plain implementation."""
    from kestrel_llm_b200.csrc import ops
    ops.attention_set_small_portions(per_cent)
    try:
        _run(model_dirs, "D", "bfloat16", family, record_property, lengths=LENGTHS_MIXED["D"] if family is R.trace_mixed else None)
    finally:
        ops.attention_set_small_portions()


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", DTYPES)
def test_cuttings_agree_with_each_other(model_dirs, name, dtype):
    """Beyond the comparison with the plain implementation: the same position's logits from
    different cuttings.  In float32 every kernel fixes the order of each output's sums
    whatever the batch, the cut and the pages, so the logits are the same BITS under all four
    families and from captured steps (the reference's own criterion is identity too,
    src/main.c:2207-2213); in bfloat16 kernels are picked by the number of tokens, and the
    logits differ by rounding only."""
    reqs = _requests(name)
    results = []
    for family, graphs in ((R.trace_whole, False), (R.trace_tail_decode, False), (R.trace_portions, False),
                           (R.trace_mixed, False), (R.trace_tail_decode, True), (R.trace_mixed, True)):
        steps, max_tokens = family(reqs)
        results.append(R.run_trace(R.make_engine(model_dirs[name][dtype], dtype, max_tokens, graphs=graphs), steps))
    for k, other in enumerate(results[1:], 1):
        for rname, toks in reqs.items():
            scale = max(float(np.abs(results[0][rname][p]).max()) for p in range(len(toks)))
            for p in range(len(toks)):
                if dtype == "float32":
                    assert np.array_equal(other[rname][p], results[0][rname][p]), \
                        f"cutting {k}: request {rname} position {p}: float32 logits differ by " \
                        f"{np.abs(other[rname][p] - results[0][rname][p]).max():.3e}"
                else:
                    err = float(np.abs(other[rname][p] - results[0][rname][p]).max()) / scale
                    assert err <= 2e-2, f"cutting {k}: request {rname} position {p}: cuttings differ by {err:.3e}"


@pytest.mark.parametrize("graphs", [1, 0])
@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_run_program(model_dirs, dtype, graphs, tmp_path):
    """bin/trace_run as a user calls it: JSON lines in, <step>.f32 files and `done` lines out;
    with decode steps replayed from captured graphs (the default, what generation runs) and
    launched kernel by kernel."""
    name = "A"
    reqs = _requests(name)
    steps, max_tokens = R.trace_mixed(reqs, seed=3)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    lines = "".join(json.dumps(dict(step=i, **s)) + "\n" for i, s in enumerate(steps))
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", model_dirs[name][dtype],
                        "--dtype", dtype, "--out", str(out), "--max-tokens", str(max_tokens), "--cuda-graphs", str(graphs)],
                       input=lines, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(len(steps))]
    V = tiny_configs.A["vocab_size"]
    pos = {n: 0 for n in reqs}
    got = {n: {} for n in reqs}
    for i, s in enumerate(steps):
        arr = np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, V)
        r = 0
        for e in s["entries"]:
            for w in e["want"]:
                got[e["id"]][pos[e["id"]] + w] = arr[r]
                r += 1
            pos[e["id"]] += len(e["tokens"])
        assert r == arr.shape[0]
    R.compare_with_plain(model_dirs[name]["float32"], reqs, got, dtype, f"trace_run/{dtype}")
