"""Plain restatement of the Qwen3 dense decoder, for tests only.

Whole sequences, no cache, no batching, one function per part, numpy float32 throughout.
Nothing here is imported by the engine and nothing of the engine is imported here: the file
has its own config reader and its own safetensors reader so that a fault in the product's
loader cannot cancel out in a comparison.

Every function cites the lines of the reference (paths inside the kestrel-llm project) whose
formula it restates.  ``src/model/vllm_safetensors.c`` is abbreviated ``st.c``.
"""
from __future__ import annotations

import json
import os
import struct

import numpy as np

F32 = np.float32


# ----------------------------------------------------------------------------------------------
# reading a model folder (independent of the engine's loader)
# ----------------------------------------------------------------------------------------------

def read_config(model_dir: str) -> dict:
    """config.json keys as the reference's converter reads them
    (vqf_convert/src/model_cfgio.c:259-291): hidden_size, num_hidden_layers,
    num_attention_heads, num_key_value_heads, intermediate_size, vocab_size, rope_theta,
    rms_norm_eps, head_dim (falls back to hidden/heads).  attention_bias,
    tie_word_embeddings and the sliding-window keys are not read by the reference; their
    meaning here follows the checkpoint format the reference converts."""
    with open(os.path.join(model_dir, "config.json")) as f:
        raw = json.load(f)
    c = dict(raw)
    c.setdefault("num_key_value_heads", c["num_attention_heads"])
    if not c.get("head_dim"):
        c["head_dim"] = c["hidden_size"] // c["num_attention_heads"]
    c.setdefault("rope_theta", 10000.0)
    c.setdefault("rms_norm_eps", 1e-6)
    c.setdefault("attention_bias", False)
    c.setdefault("tie_word_embeddings", False)
    return c


def read_safetensors(path: str) -> dict:
    """All tensors of one .safetensors file as float32 numpy arrays (integers stay integers).

    Format as parsed by vqf_convert/src/model_cfgio.c:167-200: u64 little-endian header
    length, JSON header {name: {dtype, shape, data_offsets}}, then raw bytes.  BF16 widens by
    a 16-bit shift (model_cfgio.c:688-701)."""
    with open(path, "rb") as f:
        blob = f.read()
    (hlen,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + hlen].decode("utf-8"))
    base = 8 + hlen
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        raw = blob[base + b: base + e]
        dt = info["dtype"]
        shape = tuple(info["shape"])
        if dt == "BF16":
            u16 = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            arr = u16.view(np.float32)
        elif dt == "F16":
            arr = np.frombuffer(raw, dtype="<f2").astype(np.float32)
        elif dt == "F32":
            arr = np.frombuffer(raw, dtype="<f4").astype(np.float32)
        elif dt == "I32":
            arr = np.frombuffer(raw, dtype="<i4")
        elif dt == "I64":
            arr = np.frombuffer(raw, dtype="<i8")
        else:
            raise ValueError(f"plain reader: dtype {dt} of {name}")
        out[name] = arr.reshape(shape).copy()
    return out


def read_model(model_dir: str):
    return read_config(model_dir), read_safetensors(os.path.join(model_dir, "model.safetensors"))


# ----------------------------------------------------------------------------------------------
# parts
# ----------------------------------------------------------------------------------------------

def embedding(table: np.ndarray, tokens) -> np.ndarray:
    """x = E[token] (st.c:16392-16393)."""
    return table[np.asarray(tokens, dtype=np.int64)].astype(F32)


def rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """ss = sum x^2; r = 1/sqrtf(ss/d + eps); out = (x*r)*w over the last axis
    (st.c:8811-8827; batch form st.c:8848-8867)."""
    x = x.astype(F32)
    d = x.shape[-1]
    ss = np.sum(x * x, axis=-1, keepdims=True, dtype=F32)
    r = (F32(1.0) / np.sqrt(ss / F32(d) + F32(eps))).astype(F32)
    return ((x * r) * w.astype(F32)).astype(F32)


def linear(x: np.ndarray, w: np.ndarray, b=None) -> np.ndarray:
    """y[r] = sum_c W[r,c] x[c], weights [out,in] used without transpose
    (st.c:8880-8892).  A bias, where the checkpoint has one, is added after the product."""
    y = x.astype(F32) @ w.astype(F32).T
    if b is not None:
        y = y + b.astype(F32)
    return y.astype(F32)


def head_rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """Per-head norm over head_dim, one weight vector shared by all heads of a layer
    (st.c:9541-9561, batched st.c:16941-16959).  x: [T, heads, hd].  The reference writes
    the literal 1e-6f here; the caller passes the value."""
    return rms_norm(x, w, eps)


def rope_angles(positions, head_dim: int, theta: float):
    """half = hd/2; f_j = 1/powf(theta, j/half); angle = (float)pos * f_j
    (st.c:8937-8948, st.c:8969-8971).  Returns cos, sin of shape [T, half] in float32."""
    half = head_dim // 2
    j = np.arange(half, dtype=F32)
    freq = (F32(1.0) / np.power(F32(theta), j / F32(half), dtype=F32)).astype(F32)
    ang = (np.asarray(positions, dtype=F32)[:, None] * freq[None, :]).astype(F32)
    return np.cos(ang).astype(F32), np.sin(ang).astype(F32)


def rope(x: np.ndarray, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """Rotate-half pairing (j, j+half): x_j' = x_j c - x_{j+half} s;
    x_{j+half}' = x_{j+half} c + x_j s, all head_dim dims (st.c:8972-8989).
    x: [T, heads, hd]."""
    half = x.shape[-1] // 2
    a = x[..., :half]
    b = x[..., half:]
    c = cos[:, None, :]
    s = sin[:, None, :]
    return np.concatenate([a * c - b * s, b * c + a * s], axis=-1).astype(F32)


def causal_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, window: int = 0) -> np.ndarray:
    """q [T, nh, hd], k/v [T, nkv, hd] -> [T, nh, hd].

    kh = (h*nkv)/nh (st.c:10782); scale = 1/sqrtf(hd) (st.c:16549); score = dot*scale
    (st.c:10846); the mask is the loop bound, keys 0..t (st.c:1974); p = expf(s - max),
    w = p/sum (st.c:10852-10856, 10898); out = sum_s w_s V_s in ascending s
    (st.c:10896-10910).  `window` > 0 keeps only the last `window` keys (t-window+1..t); the
    reference has no such option, the checkpoint format does."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    scale = F32(1.0) / np.sqrt(F32(hd))
    out = np.zeros((T, nh, hd), dtype=F32)
    for h in range(nh):
        kh = (h * nkv) // nh
        for t in range(T):
            lo = 0 if window <= 0 else max(0, t - window + 1)
            ks = k[lo:t + 1, kh, :]
            vs = v[lo:t + 1, kh, :]
            sc = (ks @ q[t, h, :]).astype(F32) * scale
            m = np.max(sc)
            p = np.exp(sc - m, dtype=F32)
            wgt = (p / np.sum(p, dtype=F32)).astype(F32)
            out[t, h, :] = wgt @ vs
    return out


def silu(z: np.ndarray) -> np.ndarray:
    """silu(z) = z / (1 + expf(-z)) (st.c:3605-3607)."""
    z = z.astype(F32)
    return (z / (F32(1.0) + np.exp(-z, dtype=F32))).astype(F32)


def gated_mlp(x: np.ndarray, wg: np.ndarray, wu: np.ndarray, wd: np.ndarray) -> np.ndarray:
    """g = Wg x; u = Wu x; a = silu(g)*u; y = Wd a (st.c:8904-8914)."""
    g = linear(x, wg)
    u = linear(x, wu)
    return linear((silu(g) * u).astype(F32), wd)


def attention_block(x, positions, P, cfg, layer, window=0):
    """Rows 3-8 of the layer: projections (st.c:16440-16442), per-head QK norm
    (st.c:16466-16475), RoPE (st.c:16485), attention, output projection."""
    T = x.shape[0]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    pre = f"model.layers.{layer}.self_attn."
    bias = cfg["attention_bias"]
    q = linear(x, P[pre + "q_proj.weight"], P.get(pre + "q_proj.bias") if bias else None)
    k = linear(x, P[pre + "k_proj.weight"], P.get(pre + "k_proj.bias") if bias else None)
    v = linear(x, P[pre + "v_proj.weight"], P.get(pre + "v_proj.bias") if bias else None)
    q = q.reshape(T, nh, hd)
    k = k.reshape(T, nkv, hd)
    v = v.reshape(T, nkv, hd)
    qk_eps = cfg.get("qk_norm_eps", cfg["rms_norm_eps"])
    if pre + "q_norm.weight" in P:
        q = head_rms_norm(q, P[pre + "q_norm.weight"], qk_eps)
        k = head_rms_norm(k, P[pre + "k_norm.weight"], qk_eps)
    cos, sin = rope_angles(positions, hd, cfg["rope_theta"])
    q = rope(q, cos, sin)
    k = rope(k, cos, sin)
    a = causal_attention(q, k, v, window).reshape(T, nh * hd)
    return linear(a, P[pre + "o_proj.weight"], P.get(pre + "o_proj.bias") if bias else None)


def layer_window(cfg: dict, layer: int) -> int:
    """Window of a layer, 0 for full attention.  ``layer_types`` wins; else layers from
    ``max_window_layers`` on are windowed when ``use_sliding_window`` is set."""
    sw = cfg.get("sliding_window")
    if not sw:
        return 0
    lt = cfg.get("layer_types")
    if lt:
        return int(sw) if lt[layer] == "sliding_attention" else 0
    if cfg.get("use_sliding_window") and layer >= int(cfg.get("max_window_layers", 0)):
        return int(sw)
    return 0


def decoder_layer(x, positions, P, cfg, layer):
    """res = x; n = norm(x); x = res + attn(n) (st.c:16412-16413, 16622-16626);
    res = x; n = norm(x); x = res + mlp(n) (st.c:16704-16705, 16796-16797)."""
    pre = f"model.layers.{layer}."
    eps = cfg["rms_norm_eps"]
    n = rms_norm(x, P[pre + "input_layernorm.weight"], eps)
    x = (x + attention_block(n, positions, P, cfg, layer, layer_window(cfg, layer))).astype(F32)
    n = rms_norm(x, P[pre + "post_attention_layernorm.weight"], eps)
    y = gated_mlp(n, P[pre + "mlp.gate_proj.weight"], P[pre + "mlp.up_proj.weight"],
                  P[pre + "mlp.down_proj.weight"])
    return (x + y).astype(F32)


def forward_logits(cfg: dict, P: dict, tokens) -> np.ndarray:
    """Logits [T, V] of one whole sequence: embedding, the layers in order, final norm
    (st.c:16834), lm_head (st.c:16850-16855).  With tied embeddings, or when the file has no
    lm_head, the embedding table is the head (vqf_convert/src/conv_main.c:613-614,
    1015-1020)."""
    tokens = list(tokens)
    positions = np.arange(len(tokens))
    x = embedding(P["model.embed_tokens.weight"], tokens)
    for layer in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, positions, P, cfg, layer)
    n = rms_norm(x, P["model.norm.weight"], cfg["rms_norm_eps"])
    head = P["model.embed_tokens.weight"] if (cfg["tie_word_embeddings"] or "lm_head.weight" not in P) \
        else P["lm_head.weight"]
    return linear(n, head)


# ----------------------------------------------------------------------------------------------
# sampling (src/core/vllm_transformer.c:357-479), deterministic given the uniform number
# ----------------------------------------------------------------------------------------------

def greedy(logits: np.ndarray) -> int:
    """First maximum wins: strict > scan from index 0 (vllm_transformer.c:362-367)."""
    best = 0
    for i in range(1, logits.shape[0]):
        if logits[i] > logits[best]:
            best = i
    return best


def repetition_penalty(logits: np.ndarray, generated, penalty: float, window: int = 32) -> np.ndarray:
    """The streaming harness's penalty (src/main.c:3741-3752 options, 3768-3782 loop): a copy of
    the logits in which, for each of the last ``window`` generated tokens, most recent first, the
    token's logit l is replaced by l / penalty if l >= 0, else l * penalty - once per occurrence."""
    out = np.array(logits, dtype=F32, copy=True)
    if not penalty > 1.0:
        return out
    cnt = min(len(generated), window)
    for h in range(cnt):
        tid = generated[len(generated) - 1 - h]
        if tid < 0 or tid >= out.shape[0]:
            continue
        l = out[tid]
        out[tid] = F32(l / F32(penalty)) if l >= 0 else F32(l * F32(penalty))
    return out


def sample_probs(logits: np.ndarray, temperature: float, top_k: int = 0, min_p: float = 0.0,
                 top_p: float = 1.0) -> np.ndarray:
    """Filtered, unnormalised probabilities in the reference's order: softmax((l-max)/T)
    (vllm_transformer.c:393-404), top-k (:313-355, :413), min-p against the largest
    probability (:418-423), top-p = shortest descending prefix whose mass reaches top_p, ties
    by lower index (:426-458).  The reference also zeroes ids 0, 1 and 3 (:406-409), a
    leftover of its toy tokenizer that the engine does not copy."""
    l = logits.astype(F32)
    p = np.exp((l - np.max(l)) / F32(temperature), dtype=F32)
    p = (p / np.sum(p, dtype=F32)).astype(F32)
    V = p.shape[0]
    order = np.lexsort((np.arange(V), -p))  # descending probability, ascending index
    if 0 < top_k < V:
        keep = np.zeros(V, dtype=bool)
        keep[order[:top_k]] = True
        p = np.where(keep, p, F32(0))
    if min_p > 0:
        p = np.where(p < F32(min_p) * np.max(p), F32(0), p)
    if top_p < 1.0:
        order = np.lexsort((np.arange(V), -p))
        cum = F32(0)
        keep = np.zeros(V, dtype=bool)
        for idx in order:
            if not cum < F32(top_p):
                break
            keep[idx] = True
            cum = F32(cum + p[idx])
        p = np.where(keep, p, F32(0))
    return p.astype(F32)


def sample_from(p: np.ndarray, u: float) -> int:
    """r = u * sum p; first i whose running sum reaches r (vllm_transformer.c:464-471)."""
    r = F32(u) * np.sum(p, dtype=F32)
    c = np.cumsum(p, dtype=F32)
    idx = int(np.searchsorted(c, r, side="left"))
    return min(idx, p.shape[0] - 1)
