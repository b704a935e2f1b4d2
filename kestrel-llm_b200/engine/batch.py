"""The description of one step's tokens, on the host and on the device.

A step runs a flat list of T tokens from ``nseq`` requests: prompt portions (several tokens of
one request, in order) beside single decoded tokens.  Everything a kernel needs to place a
token - its id, its position in its request, which request, that request's pages - is packed
by the native host runtime (`kbatch_pack`, csrc/host/batch_pack.cpp) into one int32 buffer and
copied to the device in one transfer.  Only generic facts are in it; what a kernel derives from
them (tiles, slices) is made by the part that owns the kernel, from the host copy (``host``,
``layout``).
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheError, host_library
from ..csrc import cdecl as _cdecl

_K = _cdecl.constants()
LAYOUT_INTS = _K["KBATCH_LAYOUT_INTS"]

# Every step has a serial of its own, by which parts recognise that what they derived from the
# last description is stale.  The native runner counts its steps from 1; these start far above.
_serials = itertools.count(1 << 40)


def next_serial() -> int:
    return next(_serials)


@dataclass
class Entry:
    """Tokens [start, start + len(tokens)) of request ``rid``; ``want`` lists the offsets among
    these tokens whose logits are asked for."""
    rid: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


def flatten(entries: Sequence[Entry]):
    """The entries as the flat arrays the native runtime takes: request ids (int64), token
    counts, all token ids one after the other, wanted places per entry and all wanted offsets
    (int32)."""
    n = len(entries)
    ids = np.fromiter((e.rid for e in entries), dtype=np.int64, count=n)
    counts = np.fromiter((len(e.tokens) for e in entries), dtype=np.int32, count=n)
    if n == 1:
        tokens = np.asarray(entries[0].tokens, dtype=np.int32)
    else:
        tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int32) for e in entries])
    want_counts = np.fromiter((len(e.want) for e in entries), dtype=np.int32, count=n)
    wants = np.fromiter((int(w) for e in entries for w in e.want), dtype=np.int32)
    return ids, counts, np.ascontiguousarray(tokens), want_counts, wants


class StepBatch:
    """One step's description as tensors, for parts whose forward pass runs from Python."""

    captured = False            # launches made with it are not being recorded for replay

    def __init__(self, entries: Sequence[Entry], cache, device, table_width: Optional[int] = None):
        """``cache`` is the `CacheManager`; pages for every entry must be reserved already."""
        lib = host_library()
        self.entries = list(entries)
        ids, counts, tokens, want_counts, wants = flatten(entries)
        n = len(entries)
        need = lib.kbatch_ints_needed(cache.handle, n, ids.ctypes.data, counts.ctypes.data, int(wants.shape[0]), table_width or 0)
        if need < 0:
            raise CacheError(f"cannot describe the step (code {need}): a request is not live, or an entry is empty")
        pinned = torch.empty(need, dtype=torch.int32)
        if torch.device(device).type == "cuda":
            pinned = pinned.pin_memory()
        host = pinned.numpy()
        layout = np.zeros(LAYOUT_INTS, dtype=np.int32)
        total = lib.kbatch_pack(cache.handle, n, ids.ctypes.data, counts.ctypes.data, tokens.ctypes.data, want_counts.ctypes.data,
                                wants.ctypes.data, table_width or 0, host.ctypes.data, need, layout.ctypes.data)
        if total < 0:
            if total == -2:
                raise ValueError("a wanted place lies outside its entry's tokens of this step")
            raise CacheError(f"cannot describe the step (code {total})")
        self.host, self.layout = host, layout
        self.serial = next_serial()
        T, R, W = int(layout[_K["KB_NUM_TOKENS"]]), int(layout[_K["KB_NUM_ROWS"]]), int(layout[_K["KB_TABLE_WIDTH"]])
        G = int(layout[_K["KB_NUM_GROUPS"]])
        self.num_tokens, self.num_seqs, self.num_logit_rows, self.table_width = T, n, R, W
        dev = pinned.to(device, non_blocking=True)
        self._pinned = pinned            # keep alive until the copy has run
        self.device_buffer = dev

        def section(name: str, length: int) -> torch.Tensor:
            o = int(layout[_K[name]])
            return dev[o:o + length]

        self.token_ids = section("KB_O_TOKEN_IDS", T)
        self.positions = section("KB_O_POSITIONS", T)
        self.seq_of_token = section("KB_O_SEQ_OF_TOKEN", T)
        self.cu_seqlens = section("KB_O_CU_SEQLENS", n + 1)
        self.kv_lens = section("KB_O_KV_LENS", n)
        self.slots = section("KB_O_SLOTS", n)
        self.logit_rows = section("KB_O_ROWS", R)
        self._tables = [section("KB_O_TABLES", G * n * W)[g * n * W:(g + 1) * n * W].view(n, W) for g in range(G)]
        o_cu, o_kv, o_slot = int(layout[_K["KB_O_CU_SEQLENS"]]), int(layout[_K["KB_O_KV_LENS"]]), int(layout[_K["KB_O_SLOTS"]])
        self.counts = counts.tolist()
        self.cu_seqlens_host = host[o_cu:o_cu + n + 1].tolist()
        self.kv_lens_host = host[o_kv:o_kv + n].tolist()
        self.slots_host = host[o_slot:o_slot + n].tolist()
        self.starts = [k - c for k, c in zip(self.kv_lens_host, self.counts)]
        self.max_count = int(layout[_K["KB_MAX_COUNT"]])
        self.max_kv_len = int(layout[_K["KB_MAX_KV_LEN"]])
        self.bytes_h2d = int(total) * 4

    def block_table(self, group: int) -> torch.Tensor:
        return self._tables[group]

    @property
    def is_decode_only(self) -> bool:
        return self.max_count == 1
