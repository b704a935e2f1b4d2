"""The description of one step's tokens, on the host and on the device.

A step runs a flat list of T tokens from ``nseq`` requests: prompt portions (several tokens of
one request, in order) beside single decoded tokens.  Everything a kernel needs to place a
token - its id, its position in its request, which request, that request's pages - is packed
into one int32 buffer on the host and copied to the device in one transfer.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch


@dataclass
class Entry:
    """Tokens [start, start + len(tokens)) of request ``rid``; ``want`` lists the offsets among
    these tokens whose logits are asked for."""
    rid: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class TileList:
    """Tiles of the tensor-core attention kernel: request and first row of each tile (device
    int32), their number and the longest request among them.  ``slice_len_table``, set only
    for a captured decode step, is a device table whose entry s is the slice length to use
    with s slices."""
    seq: torch.Tensor
    row0: torch.Tensor
    count: int
    max_kv: int
    slice_len_table: Optional[torch.Tensor] = None


@dataclass
class AttentionPlan:
    """Tile lists for requests with few rows (at most 16 per kv head: decode tokens) and for
    the others (prompt portions); None where there are none."""
    small: Optional[TileList]
    large: Optional[TileList]


class StepBatch:
    def __init__(self, entries: Sequence[Entry], cache, device, table_width: Optional[int] = None):
        """``cache`` is the `CacheManager`; pages for every entry must be reserved already."""
        nseq = len(entries)
        counts = [len(e.tokens) for e in entries]
        T = int(sum(counts))
        self.num_tokens, self.num_seqs = T, nseq
        self.entries = list(entries)
        starts = [cache.length(e.rid) for e in entries]
        self.starts = starts
        self.kv_lens_host = [s + c for s, c in zip(starts, counts)]
        rows: List[int] = []
        off = 0
        for e, c in zip(entries, counts):
            for w in e.want:
                if not 0 <= w < c:
                    raise ValueError(f"request {e.rid}: wanted place {w} outside its {c} tokens of this step")
                rows.append(off + w)
            off += c
        R = len(rows)
        self.num_logit_rows = R
        n_groups = cache.num_groups
        if table_width is None:
            need = 1
            for g in range(n_groups):
                for e in entries:
                    need = max(need, cache.num_blocks(e.rid, g))
            table_width = (need + 7) // 8 * 8
        self.table_width = table_width
        # layout of the packed buffer
        o_tok, o_pos, o_seq = 0, T, 2 * T
        o_cu = 3 * T
        o_kv = o_cu + nseq + 1
        o_slot = o_kv + nseq
        o_rows = o_slot + nseq
        o_tab = o_rows + R
        total = o_tab + n_groups * nseq * table_width
        host = np.empty(max(total, 1), dtype=np.int32)
        cu = 0
        for i, (e, c, s) in enumerate(zip(entries, counts, starts)):
            host[o_tok + cu:o_tok + cu + c] = np.asarray(e.tokens, dtype=np.int64)
            host[o_pos + cu:o_pos + cu + c] = np.arange(s, s + c, dtype=np.int32)
            host[o_seq + cu:o_seq + cu + c] = i
            host[o_cu + i] = cu
            host[o_kv + i] = s + c
            host[o_slot + i] = cache.slot(e.rid)
            cu += c
        host[o_cu + nseq] = cu
        host[o_rows:o_rows + R] = rows
        for g in range(n_groups):
            for i, e in enumerate(entries):
                b = o_tab + (g * nseq + i) * table_width
                cache.block_table_into(e.rid, g, host[b:b + table_width])
        self.host = host
        pinned = torch.from_numpy(host)
        if torch.device(device).type == "cuda":
            pinned = pinned.pin_memory()
        dev = pinned.to(device, non_blocking=True)
        self._pinned = pinned            # keep alive until the copy has run
        self.device_buffer = dev
        self.token_ids = dev[o_tok:o_tok + T]
        self.positions = dev[o_pos:o_pos + T]
        self.seq_of_token = dev[o_seq:o_seq + T]
        self.cu_seqlens = dev[o_cu:o_cu + nseq + 1]
        self.kv_lens = dev[o_kv:o_kv + nseq]
        self.slots = dev[o_slot:o_slot + nseq]
        self.logit_rows = dev[o_rows:o_rows + R]
        self._tables = [dev[o_tab + g * nseq * table_width: o_tab + (g + 1) * nseq * table_width]
                        .view(nseq, table_width) for g in range(n_groups)]
        self.counts = counts
        self.cu_seqlens_host = [int(x) for x in host[o_cu:o_cu + nseq + 1]]
        self.slots_host = [int(x) for x in host[o_slot:o_slot + nseq]]
        self.max_count = max(counts) if counts else 0
        self.max_kv_len = max(self.kv_lens_host) if counts else 0
        self.bytes_h2d = int(host.nbytes)
        self._plans = {}

    def attention_plan(self, group_size: int, rows_large: int = 64) -> "AttentionPlan":
        """How the tensor-core attention kernel tiles this step's rows for mixers with
        ``group_size`` query heads per kv head: requests with at most 16 rows (token, head) go
        into tiles of 16 rows, the others into tiles of ``rows_large``.  Built once per step and
        (group size, tile size); the tile lists are a second, small copy to the device."""
        plan = self._plans.get((group_size, rows_large))
        if plan is None:
            small_s, small_r, large_s, large_r = [], [], [], []
            small_kv = large_kv = 0
            for i, c in enumerate(self.counts):
                rows = c * group_size
                if rows <= 16:
                    small_s.append(i)
                    small_r.append(0)
                    small_kv = max(small_kv, self.kv_lens_host[i])
                else:
                    for r0 in range(0, rows, rows_large):
                        large_s.append(i)
                        large_r.append(r0)
                    large_kv = max(large_kv, self.kv_lens_host[i])
            flat = np.asarray(small_s + small_r + large_s + large_r, dtype=np.int32)
            dev = torch.from_numpy(flat)
            if self.device_buffer.is_cuda:
                dev = dev.pin_memory()
            dev = dev.to(self.device_buffer.device, non_blocking=True)
            ns, nl = len(small_s), len(large_s)
            self.bytes_h2d += int(flat.nbytes)
            plan = AttentionPlan(
                TileList(dev[:ns], dev[ns:2 * ns], ns, small_kv) if ns else None,
                TileList(dev[2 * ns:2 * ns + nl], dev[2 * ns + nl:], nl, large_kv) if nl else None)
            self._plans[(group_size, rows_large)] = plan
        return plan

    def block_table(self, group: int) -> torch.Tensor:
        return self._tables[group]

    @property
    def is_decode_only(self) -> bool:
        return self.max_count == 1
