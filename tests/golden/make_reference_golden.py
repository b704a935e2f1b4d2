"""Makes tests/golden/reference_logits_<name>.npy: logits of the REFERENCE's own compiled float32
forward pass on the tiny random models in tests/golden/tiny_model_<name>, for two
configurations that differ in every size.

    python tests/golden/make_reference_golden.py /path/to/kestrel-llm

It compiles six of the reference's C files with gcc on the CPU (the float32 fallback of
src/model/vllm_safetensors.c needs no ARM board), links them with reference_harness.c and
reference_stubs.c, feeds the model's weights and the token ids below through
st_qwen_model_forward one token at a time with VLLM_KV_F32=1 (without it the reference keeps
an int8 shadow of the cache and reads that), and stores the logits after every token.
tests/test_plain_reference.py compares tests/plain_qwen3.py with the stored file, so the
plain implementation is anchored on the reference's code, not only on its formulas.

Each request is 100 tokens long: from 64 keys on the reference's float32 attention switches
from its plain loop to the tiled online-softmax kernel (src/model/vllm_safetensors.c:16556-16562,
9762-9859), so both of its attention paths are the oracle.

Limits of the anchor: one token at a time only; no attention bias; the per-head norm's eps is
the literal 1e-6 of the reference.  The model folders are written by this script as well (numpy
generator, seeds below) so that each pair stays consistent.
"""
import json
import os
import struct
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
BASE = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", max_position_embeddings=256, rms_norm_eps=1e-6,
            hidden_act="silu", tie_word_embeddings=False, attention_bias=False, torch_dtype="bfloat16")
# name -> (configuration, seed of the weights, seed of the tokens)
CONFIGS = {
    "a": (dict(BASE, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
               intermediate_size=48, vocab_size=64, rope_theta=1000000.0), 7, 70),
    "b": (dict(BASE, hidden_size=96, num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=2, head_dim=32,
               intermediate_size=200, vocab_size=509, rope_theta=1000000.0), 8, 80),
}
N_TOKENS = 100


def bf16_round(a):
    u = a.astype(np.float32).view(np.uint32)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.view(np.float32)


def make_weights(c, seed):
    rng = np.random.default_rng(seed)
    d, L, nh, nkv, hd, ff, V = (c["hidden_size"], c["num_hidden_layers"], c["num_attention_heads"],
                                c["num_key_value_heads"], c["head_dim"], c["intermediate_size"], c["vocab_size"])
    W = {}

    def lin(name, *shape):
        W[name] = bf16_round(rng.normal(0, 0.05, shape))

    def nrm(name, n):
        W[name] = bf16_round(1 + rng.normal(0, 0.05, (n,)))

    lin("model.embed_tokens.weight", V, d)
    for l in range(L):
        p = f"model.layers.{l}."
        nrm(p + "input_layernorm.weight", d)
        lin(p + "self_attn.q_proj.weight", nh * hd, d)
        lin(p + "self_attn.k_proj.weight", nkv * hd, d)
        lin(p + "self_attn.v_proj.weight", nkv * hd, d)
        lin(p + "self_attn.o_proj.weight", d, nh * hd)
        nrm(p + "self_attn.q_norm.weight", hd)
        nrm(p + "self_attn.k_norm.weight", hd)
        nrm(p + "post_attention_layernorm.weight", d)
        lin(p + "mlp.gate_proj.weight", ff, d)
        lin(p + "mlp.up_proj.weight", ff, d)
        lin(p + "mlp.down_proj.weight", d, ff)
    nrm("model.norm.weight", d)
    lin("lm_head.weight", V, d)
    return W


def write_safetensors_bf16(path, W):
    header, off, blobs = {}, 0, []
    for n, a in W.items():
        b = (a.astype(np.float32).view(np.uint32) >> 16).astype("<u2").tobytes()
        header[n] = {"dtype": "BF16", "shape": list(a.shape), "data_offsets": [off, off + len(b)]}
        off += len(b)
        blobs.append(b)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def build_probe(ref, tmp):
    """Compiles the reference's model code and the harness; returns the executable."""
    incs = [f"-I{ref}/include/{d}" for d in ("common", "core", "serve", "model", "npu", "npu/rk3588", "media")]
    incs.append(f"-I{ref}/src/model")
    flags = "-std=gnu11 -O1 -D_GNU_SOURCE -mavx2 -mfma -ffp-contract=off -pthread -fopenmp -w".split()
    objs = []
    for src in ("src/model/vllm_safetensors.c", "src/core/vllm_tp.c", "src/core/vllm_l3.c", "src/core/vllm_ep.c",
                "src/model/vqf.c", "src/common/vllm_crypto.c"):
        o = os.path.join(tmp, os.path.basename(src)[:-2] + ".o")
        subprocess.run(["gcc"] + flags + incs + ["-c", os.path.join(ref, src), "-o", o], check=True)
        objs.append(o)
    for src in ("reference_harness.c", "reference_stubs.c"):
        o = os.path.join(tmp, src[:-2] + ".o")
        subprocess.run(["gcc"] + flags + incs + ["-c", os.path.join(HERE, src), "-o", o], check=True)
        objs.append(o)
    exe = os.path.join(tmp, "probe")
    subprocess.run(["gcc", "-o", exe] + objs + ["-lm", "-pthread", "-fopenmp", "-ldl"], check=True)
    return exe


def run_one(exe, tmp, name, c, wseed, tseed):
    W = make_weights(c, wseed)
    tokens = np.random.default_rng(tseed).integers(0, c["vocab_size"], size=N_TOKENS).tolist()
    mdir = os.path.join(HERE, f"tiny_model_{name}")
    os.makedirs(mdir, exist_ok=True)
    with open(os.path.join(mdir, "config.json"), "w") as f:
        json.dump(c, f, indent=1)
    write_safetensors_bf16(os.path.join(mdir, "model.safetensors"), W)
    L = c["num_hidden_layers"]
    flat = os.path.join(tmp, f"in_{name}.bin")
    with open(flat, "wb") as f:
        f.write(struct.pack("<8i", L, c["hidden_size"], c["num_attention_heads"], c["num_key_value_heads"],
                            c["head_dim"], c["intermediate_size"], c["vocab_size"], len(tokens)))
        f.write(struct.pack("<2f", c["rope_theta"], c["rms_norm_eps"]))
        f.write(struct.pack(f"<{len(tokens)}i", *tokens))

        def put(a):
            f.write(np.ascontiguousarray(a, dtype="<f4").tobytes())

        def stack(suffix):
            return np.concatenate([W[f"model.layers.{l}.{suffix}"].reshape(-1) for l in range(L)])

        put(W["model.embed_tokens.weight"]); put(W["lm_head.weight"]); put(W["model.norm.weight"])
        for s in ("input_layernorm.weight", "post_attention_layernorm.weight", "self_attn.q_proj.weight",
                  "self_attn.k_proj.weight", "self_attn.v_proj.weight", "self_attn.o_proj.weight",
                  "self_attn.q_norm.weight", "self_attn.k_norm.weight", "mlp.gate_proj.weight",
                  "mlp.up_proj.weight", "mlp.down_proj.weight"):
            put(stack(s))
    out = os.path.join(tmp, f"out_{name}.bin")
    env = dict(os.environ, VLLM_KV_F32="1", VLLM_THREADS="1", OMP_NUM_THREADS="1")
    subprocess.run([exe, flat, out], check=True, env=env, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    logits = np.fromfile(out, dtype="<f4").reshape(len(tokens), c["vocab_size"])
    np.save(os.path.join(HERE, f"reference_logits_{name}.npy"), logits)
    with open(os.path.join(HERE, f"reference_tokens_{name}.json"), "w") as f:
        json.dump(tokens, f)
    print(name, "wrote", logits.shape, "max |logit|", float(np.abs(logits).max()))


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_reference_golden.py /path/to/kestrel-llm (a checkout of the reference)")
    tmp = tempfile.mkdtemp(prefix="kestrel_golden_")
    exe = build_probe(sys.argv[1], tmp)
    for name, (c, wseed, tseed) in CONFIGS.items():
        run_one(exe, tmp, name, c, wseed, tseed)


if __name__ == "__main__":
    main()
