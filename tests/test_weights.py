"""Weights by tensor name: round trip, storage types, and the single error that lists
everything wrong with a folder (no GPU: models are built on the CPU or the meta device)."""
import json
import os
import shutil
import struct

import numpy as np
import pytest
import torch

import plain_qwen3 as P
import tiny_configs
from kestrel_llm_b200.config import Qwen3Config
from kestrel_llm_b200.weights import (ModelFolder, WeightsError, load_model, write_random_model,
                                      write_safetensors)


def _rewrite(src_dir, dst_dir, edit):
    """Copy a model folder, passing its {name: tensor} dict through `edit`."""
    os.makedirs(dst_dir, exist_ok=True)
    shutil.copy(os.path.join(src_dir, "config.json"), os.path.join(dst_dir, "config.json"))
    mf = ModelFolder(src_dir)
    tensors = {n: mf.tensor(n).clone() for n in mf.names()}
    mf.close()
    edit(tensors)
    write_safetensors(os.path.join(dst_dir, "model.safetensors"), tensors.items())
    return dst_dir


def test_random_model_round_trip(model_dirs):
    d = model_dirs["B"]["bfloat16"]
    m = load_model(d, "bfloat16", "cpu")
    cfg, W = P.read_model(d)
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    blk = m.blocks[1]
    assert blk.mixer.qkv.weight.dtype == torch.bfloat16
    np.testing.assert_array_equal(blk.mixer.qkv.weight[:q].float().numpy(), W["model.layers.1.self_attn.q_proj.weight"])
    np.testing.assert_array_equal(blk.mixer.qkv.bias[q:q + 64].numpy(), W["model.layers.1.self_attn.k_proj.bias"])
    assert blk.norm1.weight.dtype == torch.float32          # vectors are held in 32-bit
    np.testing.assert_array_equal(blk.ffn.gate_up.weight[200:].float().numpy(), W["model.layers.1.mlp.up_proj.weight"])
    np.testing.assert_array_equal(m.lm_head.weight.float().numpy(), W["lm_head.weight"])
    # distributions of the random mode
    assert abs(float(W["model.embed_tokens.weight"].std()) - 0.02) < 2e-3
    assert abs(float(W["model.norm.weight"].mean()) - 1.0) < 2e-2
    # same seed, same folder; another seed, other values
    m32 = load_model(model_dirs["B"]["float32"], "float32", "cpu")
    assert m32.blocks[0].mixer.qkv.weight.dtype == torch.float32
    np.testing.assert_array_equal(m32.blocks[0].mixer.qkv.weight.numpy(), m.blocks[0].mixer.qkv.weight.float().numpy())


def test_seed_decides_values(tmp_path):
    cfg = Qwen3Config.from_dict(tiny_configs.A)
    a = write_random_model(cfg, 0, str(tmp_path / "a"))
    b = write_random_model(cfg, 0, str(tmp_path / "b"))
    c = write_random_model(cfg, 1, str(tmp_path / "c"))
    ra, rb, rc = (open(os.path.join(d, "model.safetensors"), "rb").read() for d in (a, b, c))
    assert ra == rb and ra != rc


def test_tied_head_shares_memory(model_dirs):
    m = load_model(model_dirs["A"]["bfloat16"], "bfloat16", "cpu")
    assert m.lm_head.weight.data_ptr() == m.embedding.weight.data_ptr()
    names = [s.name for s in m.weight_slots()]
    assert "lm_head.weight" not in names


def test_one_error_lists_everything(model_dirs, tmp_path):
    def edit(t):
        del t["model.layers.0.mlp.up_proj.weight"]
        del t["model.norm.weight"]
        t["model.layers.7.extra.weight"] = torch.zeros(3, dtype=torch.bfloat16)
        t["model.layers.1.self_attn.q_proj.weight"] = torch.zeros((192, 95), dtype=torch.bfloat16)
        t["model.layers.2.self_attn.o_proj.weight"] = t["model.layers.2.self_attn.o_proj.weight"].float()
    d = _rewrite(model_dirs["B"]["bfloat16"], str(tmp_path / "bad"), edit)
    with pytest.raises(WeightsError) as e:
        load_model(d, "bfloat16", "cpu")
    msg = str(e.value)
    assert "missing tensors (2)" in msg and "model.layers.0.mlp.up_proj.weight" in msg and "model.norm.weight" in msg
    assert "unexpected tensors (1)" in msg and "model.layers.7.extra.weight" in msg
    assert "wrong shapes (1)" in msg and "[192, 95]" in msg and "[192, 96]" in msg
    assert "wrong storage types (1)" in msg and "model.layers.2.self_attn.o_proj.weight" in msg
    # the float32 engine accepts the float32 matrix, and still reports the rest
    with pytest.raises(WeightsError) as e:
        load_model(d, "float32", "cpu")
    assert "wrong storage types" not in str(e.value) and "missing tensors (2)" in str(e.value)


def test_vector_stored_in_32_bit_stays(model_dirs, tmp_path):
    w = torch.full((96,), 1.0 + 2 ** -20, dtype=torch.float32)      # not representable in bfloat16

    def edit(t):
        t["model.norm.weight"] = w
    d = _rewrite(model_dirs["B"]["bfloat16"], str(tmp_path / "v32"), edit)
    m = load_model(d, "bfloat16", "cpu")
    assert torch.equal(m.final_norm.weight, w)


def test_tied_checkpoint_may_carry_head(model_dirs, tmp_path):
    def edit(t):
        t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    d = _rewrite(model_dirs["A"]["bfloat16"], str(tmp_path / "tied"), edit)
    load_model(d, "bfloat16", "cpu")


def test_language_model_prefix_and_shards(model_dirs, tmp_path):
    src = model_dirs["A"]["bfloat16"]
    dst = tmp_path / "sharded"
    os.makedirs(dst)
    shutil.copy(os.path.join(src, "config.json"), dst / "config.json")
    mf = ModelFolder(src)
    names = mf.names()
    renamed = {("model.language_model." + n[len("model."):] if n.startswith("model.") else n): mf.tensor(n).clone()
               for n in names}
    mf.close()
    keys = sorted(renamed)
    half = len(keys) // 2
    parts = {"model-00001-of-00002.safetensors": keys[:half], "model-00002-of-00002.safetensors": keys[half:]}
    wm = {}
    for fn, ks in parts.items():
        write_safetensors(str(dst / fn), [(k, renamed[k]) for k in ks])
        wm.update({k: fn for k in ks})
    (dst / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    a = load_model(str(dst), "bfloat16", "cpu")
    b = load_model(src, "bfloat16", "cpu")
    assert torch.equal(a.blocks[1].ffn.down.weight, b.blocks[1].ffn.down.weight)
    os.remove(dst / "model.safetensors.index.json")          # third layout: shards found by name
    c = load_model(str(dst), "bfloat16", "cpu")
    assert torch.equal(c.embedding.weight, b.embedding.weight)


def test_broken_files(model_dirs, tmp_path):
    src = model_dirs["A"]["bfloat16"]
    blob = open(os.path.join(src, "model.safetensors"), "rb").read()
    for label, data, msg in (("trunc", blob[:len(blob) // 2], "outside the file"),
                             ("tiny", blob[:4], "too small"),
                             ("nohdr", struct.pack("<Q", 1 << 40) + blob[8:], "header length"),
                             ("nojson", struct.pack("<Q", 16) + b"not json at all!" + blob[24:], "not JSON")):
        d = tmp_path / label
        os.makedirs(d)
        shutil.copy(os.path.join(src, "config.json"), d / "config.json")
        (d / "model.safetensors").write_bytes(data)
        with pytest.raises(WeightsError, match=msg):
            load_model(str(d), "bfloat16", "cpu")
    (hlen,) = struct.unpack("<Q", blob[:8])
    hdr = json.loads(blob[8:8 + hlen])
    first = next(k for k in hdr if k != "__metadata__")
    hdr[first]["dtype"] = "F8_E4M3"
    hj = json.dumps(hdr).encode()
    d = tmp_path / "dtype"
    os.makedirs(d)
    shutil.copy(os.path.join(src, "config.json"), d / "config.json")
    (d / "model.safetensors").write_bytes(struct.pack("<Q", len(hj)) + hj + blob[8 + hlen:])
    with pytest.raises(WeightsError, match="unsupported dtype"):
        load_model(str(d), "bfloat16", "cpu")
    # two tensors that share bytes, and a pair of offsets in the wrong order
    hdr = json.loads(blob[8:8 + hlen])
    names = [k for k in hdr if k != "__metadata__" and hdr[k]["data_offsets"][1] > hdr[k]["data_offsets"][0]]
    size_of = lambda k: hdr[k]["data_offsets"][1] - hdr[k]["data_offsets"][0]
    a, b2 = next((x, y) for i, x in enumerate(names) for y in names[i + 1:] if size_of(x) == size_of(y))
    for label, edit, msg in (("overlap", lambda h: h[b2].__setitem__("data_offsets", list(h[a]["data_offsets"])), "overlap"),
                             ("swapped", lambda h: h[a].__setitem__("data_offsets", h[a]["data_offsets"][::-1]), "wrong order")):
        h2 = json.loads(blob[8:8 + hlen])
        edit(h2)
        hj = json.dumps(h2).encode()
        d = tmp_path / label
        os.makedirs(d)
        shutil.copy(os.path.join(src, "config.json"), d / "config.json")
        (d / "model.safetensors").write_bytes(struct.pack("<Q", len(hj)) + hj + blob[8 + hlen:])
        with pytest.raises(WeightsError, match=msg):
            load_model(str(d), "bfloat16", "cpu")
    e = tmp_path / "empty"
    os.makedirs(e)
    shutil.copy(os.path.join(src, "config.json"), e / "config.json")
    with pytest.raises(WeightsError, match="no model.safetensors"):
        load_model(str(e), "bfloat16", "cpu")
