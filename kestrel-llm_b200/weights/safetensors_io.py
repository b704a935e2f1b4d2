"""Reading and writing the safetensors container, by tensor name.

Layout (as the reference's converter parses it, vqf_convert/src/model_cfgio.c:167-200): a
little-endian u64 header length, a JSON header ``{name: {dtype, shape, data_offsets}}``, the
raw bytes.  A folder holds ``model.safetensors``, or shards listed by
``model.safetensors.index.json`` (model_cfgio.c:426-490).  Unlike the reference, an unknown
dtype, a truncated file or offsets outside the file are errors, not zeros.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from typing import Dict, Iterable, List, Tuple

import torch


class WeightsError(ValueError):
    """A model folder whose tensors do not fit the model."""


_DTYPES = {
    "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2), "F32": (torch.float32, 4),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}
_MAX_HEADER = 100 << 20


class SafetensorsFile:
    """One file, memory-mapped; tensors are views into the mapping."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise WeightsError(f"{path}: too small to be a safetensors file ({size} bytes)")
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._mm[:8])
        if hlen > _MAX_HEADER or 8 + hlen > size:
            raise WeightsError(f"{path}: header length {hlen} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._mm[8:8 + hlen].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise WeightsError(f"{path}: header is not JSON ({e})") from None
        self._base = 8 + hlen
        self.entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, info in header.items():
            if name == "__metadata__":
                continue
            dt, shape = info.get("dtype"), tuple(int(s) for s in info.get("shape", ()))
            if dt not in _DTYPES:
                raise WeightsError(f"{path}: tensor '{name}' has unsupported dtype {dt!r}")
            b, e = (int(x) for x in info["data_offsets"])
            n = 1
            for s in shape:
                n *= s
            if e < b:
                raise WeightsError(f"{path}: tensor '{name}' has its data_offsets in the wrong order ({b}, {e})")
            if b < 0 or self._base + e > size:
                raise WeightsError(f"{path}: tensor '{name}' lies outside the file "
                                   f"(offsets {b}..{e}, data section {size - self._base} bytes)")
            if e - b != n * _DTYPES[dt][1]:
                raise WeightsError(f"{path}: tensor '{name}' of shape {list(shape)} {dt} needs "
                                   f"{n * _DTYPES[dt][1]} bytes, header gives {e - b}")
            self.entries[name] = (dt, shape, b, e)
        # no byte of the data section may belong to two tensors
        spans = sorted((b, e, name) for name, (_dt, _shape, b, e) in self.entries.items() if e > b)
        for (b0, e0, n0), (b1, e1, n1) in zip(spans, spans[1:]):
            if b1 < e0:
                raise WeightsError(f"{path}: tensors '{n0}' (bytes {b0}..{e0}) and '{n1}' (bytes {b1}..{e1}) overlap")

    def names(self) -> List[str]:
        return list(self.entries)

    def info(self, name: str) -> Tuple[str, Tuple[int, ...]]:
        dt, shape, _, _ = self.entries[name]
        return dt, shape

    def tensor(self, name: str) -> torch.Tensor:
        dt, shape, b, e = self.entries[name]
        tdt, _ = _DTYPES[dt]
        if e == b:
            return torch.empty(shape, dtype=tdt)
        buf = memoryview(self._mm)[self._base + b: self._base + e]
        with warnings.catch_warnings():      # the mapping is read-only; the tensor is only read
            warnings.simplefilter("ignore", UserWarning)
            return torch.frombuffer(buf, dtype=tdt).reshape(shape)

    def close(self) -> None:
        try:
            self._mm.close()
        except BufferError:      # views still alive; the mapping goes with them
            pass
        self._f.close()


class ModelFolder:
    """All tensors of a model folder, whichever of the three layouts it uses."""

    def __init__(self, model_dir: str):
        self.dir = model_dir
        index = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        if os.path.isfile(index):
            with open(index) as f:
                wm = json.load(f).get("weight_map", {})
            shard_names = sorted(set(wm.values()))
        elif os.path.isfile(single):
            shard_names = ["model.safetensors"]
        else:
            shard_names = sorted(n for n in os.listdir(model_dir)
                                 if n.startswith("model-") and n.endswith(".safetensors"))
        if not shard_names:
            raise WeightsError(f"{model_dir}: no model.safetensors, index or shards")
        self.files = []
        self.where: Dict[str, SafetensorsFile] = {}
        for sn in shard_names:
            p = os.path.join(model_dir, sn)
            if not os.path.isfile(p):
                raise WeightsError(f"{model_dir}: shard '{sn}' named by the index is missing")
            sf = SafetensorsFile(p)
            self.files.append(sf)
            for n in sf.names():
                self.where[n] = sf

    def names(self) -> List[str]:
        return list(self.where)

    def info(self, name: str):
        return self.where[name].info(name)

    def tensor(self, name: str) -> torch.Tensor:
        return self.where[name].tensor(name)

    def close(self) -> None:
        for f in self.files:
            f.close()


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]]) -> None:
    """Write (name, tensor) pairs in the given order.  Tensors are taken one at a time so a
    large model is never held twice."""
    items = [(n, t) for n, t in tensors]
    header = {}
    off = 0
    for n, t in items:
        if t.dtype not in _NAMES:
            raise WeightsError(f"cannot store dtype {t.dtype} of '{n}'")
        nbytes = t.numel() * t.element_size()
        header[n] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for n, t in items:
            c = t.detach().contiguous().cpu()
            f.write(c.view(torch.uint8).numpy().tobytes() if c.numel() else b"")
