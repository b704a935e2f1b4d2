"""Random weights: a model folder written from a configuration and a seed, or a model filled
in place on its device.

Distributions: matrices and embeddings N(0, 0.02), norm weights 1 + N(0, 0.02), biases
N(0, 0.02).  The reference's own synthetic checkpoint (vqf_convert/test/mk_synth.py:11-37)
draws uniform values from an LCG; the normal draws here keep activations in the range real
checkpoints have.  A tensor's values depend on (seed, tensor name) only, so the folder is the
same on every machine.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Iterator, Tuple

import torch

from ..config.registry import resolve_architecture
from .loader import torch_dtype
from .safetensors_io import write_safetensors

_STD = 0.02


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def _draw(shape, init: str, gen: torch.Generator) -> torch.Tensor:
    t = torch.empty(tuple(shape), dtype=torch.float32)
    t.normal_(0.0, _STD, generator=gen)
    if init == "norm":
        t += 1.0
    return t


def write_random_model(config, seed: int, out_dir: str, dtype: str = "bfloat16") -> str:
    """Writes ``config.json`` and ``model.safetensors`` for ``config`` into ``out_dir``; every
    tensor is stored in ``dtype``.  Returns ``out_dir``."""
    store = torch_dtype(dtype)
    arch = resolve_architecture(config.architecture)
    model = arch.build(config, store, "meta")
    os.makedirs(out_dir, exist_ok=True)
    cfg = config.to_json_dict()
    cfg["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32"}[store]
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)

    def tensors() -> Iterator[Tuple[str, torch.Tensor]]:
        for slot in model.weight_slots():
            gen = torch.Generator().manual_seed(_tensor_seed(seed, slot.name))
            yield slot.name, _draw(slot.dest.shape, slot.init, gen).to(store)

    write_safetensors(os.path.join(out_dir, "model.safetensors"), tensors())
    return out_dir


def fill_random_(model, seed: int) -> None:
    """Fills a model's weights in place on its own device from the same distributions (values
    differ from `write_random_model`'s: the device's generator is used).  For sizes at which
    writing a folder first would only cost time."""
    dev = model.device
    gen = torch.Generator(device=dev).manual_seed(seed)
    with torch.no_grad():
        for slot in model.weight_slots():
            tmp = torch.empty(slot.dest.shape, dtype=torch.float32, device=dev) if slot.dest.numel() < (1 << 24) else None
            if tmp is not None:
                tmp.normal_(0.0, _STD, generator=gen)
                if slot.init == "norm":
                    tmp += 1.0
                slot.dest.copy_(tmp)
            else:
                rows = slot.dest.shape[0]
                step = max(1, (1 << 26) // max(1, slot.dest[0].numel()))
                for r in range(0, rows, step):
                    part = slot.dest[r:r + step]
                    t = torch.empty(part.shape, dtype=torch.float32, device=dev)
                    t.normal_(0.0, _STD, generator=gen)
                    if slot.init == "norm":
                        t += 1.0
                    part.copy_(t)
