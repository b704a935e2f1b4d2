"""Fills a model's weights from a folder of safetensors, by tensor name.

The model lists its `WeightSlot`s (checkpoint name -> device memory).  Every slot must be
filled by a tensor of exactly its shape; a problem of any kind - missing tensors, tensors the
model has no use for, wrong shapes, wrong storage types - is collected and reported in ONE
error, where the reference warns and continues with zeros
(vqf_convert/src/model_layers.c:45-48, vqf_convert/src/model_cfgio.c:645-648).

Storage: in bfloat16 mode matrices stay bfloat16 as stored; vectors (norm weights, biases)
are held in float32, which widens bfloat16 exactly and keeps a vector stored in 32-bit as it
is; integer tables become int32.  A matrix stored in float32 or float16 is refused in
bfloat16 mode rather than rounded silently.  In float32 mode everything widens to float32.
Names may carry the prefix ``model.language_model.`` instead of ``model.``, as the reference
accepts (model_layers.c:40-44).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.registry import architecture_of, resolve_architecture
from ..config.model_config import read_config_json
from .safetensors_io import ModelFolder, WeightsError

_TORCH_DTYPE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def torch_dtype(name: str) -> torch.dtype:
    n = {"bf16": "bfloat16", "fp32": "float32", "f32": "float32"}.get(name, name)
    if n not in _TORCH_DTYPE:
        raise ValueError(f"dtype '{name}' is not one of bfloat16, float32")
    return _TORCH_DTYPE[n]


def _alias(name: str) -> Optional[str]:
    if name.startswith("model.language_model."):
        return "model." + name[len("model.language_model."):]
    return None


def fill_from_folder(model, folder: ModelFolder) -> None:
    slots = model.weight_slots()
    wanted = {s.name: s for s in slots}
    if len(wanted) != len(slots):
        raise WeightsError("model names a checkpoint tensor twice")
    present: Dict[str, str] = {}
    for n in folder.names():
        a = _alias(n)
        present[a if (a is not None and a in wanted) else n] = n
    missing = sorted(n for n in wanted if n not in present)
    optional = set(getattr(model, "optional_tensors", ()))
    unexpected = sorted(n for n in present if n not in wanted and n not in optional)
    bad_shape: List[str] = []
    bad_dtype: List[str] = []
    for name, slot in wanted.items():
        if name not in present:
            continue
        dt, shape = folder.info(present[name])
        if tuple(shape) != tuple(slot.dest.shape):
            bad_shape.append(f"{name}: file {list(shape)}, model {list(slot.dest.shape)}")
            continue
        if slot.dest.dtype == torch.bfloat16 and dt != "BF16":
            bad_dtype.append(f"{name}: stored as {dt}; a matrix is kept as stored in bfloat16 mode "
                             f"(run with dtype float32, or convert the file)")
        elif slot.dest.dtype in (torch.float32, torch.bfloat16) and dt not in ("BF16", "F16", "F32"):
            bad_dtype.append(f"{name}: stored as {dt}, expected a floating type")
        elif slot.dest.dtype == torch.int32 and dt not in ("I32", "I64", "I16", "I8", "U8"):
            bad_dtype.append(f"{name}: stored as {dt}, expected an integer type")
    if missing or unexpected or bad_shape or bad_dtype:
        lines = [f"{folder.dir}: weights do not fit the model"]
        for title, items in (("missing tensors", missing), ("unexpected tensors", unexpected),
                             ("wrong shapes", bad_shape), ("wrong storage types", bad_dtype)):
            if items:
                lines.append(f"  {title} ({len(items)}):")
                lines += [f"    {x}" for x in items[:40]]
                if len(items) > 40:
                    lines.append(f"    ... and {len(items) - 40} more")
        raise WeightsError("\n".join(lines))
    for name, slot in wanted.items():
        src = folder.tensor(present[name])
        with torch.no_grad():
            slot.dest.copy_(src.to(slot.dest.dtype) if src.dtype != slot.dest.dtype else src)


def load_model(model_dir: str, dtype: str = "bfloat16", device="cuda:0"):
    """Model of the class that ``model_dir/config.json`` names, weights from its safetensors."""
    raw = read_config_json(model_dir)
    arch = resolve_architecture(architecture_of(raw))
    config = arch.config_class.from_dict(raw)
    model = arch.build(config, torch_dtype(dtype), device)
    folder = ModelFolder(model_dir)
    try:
        fill_from_folder(model, folder)
    finally:
        folder.close()
    return model
