"""Decode steps as CUDA graphs.

A step in which every request brings one token launches some 290 kernels at Qwen3-8B size,
each a few microseconds long; launched one by one from the host they take longer to launch
than to run.  Such a step is therefore captured - once per batch-size bucket (1, 2, 4 ... up to
``batch_max``) and class of the longest context, as two graphs of which the second is submitted
while the first runs - and replayed: the host fills ONE pinned int32 buffer (token ids,
positions, lengths, slots, the longest context, block tables) through one native call, copies
it to the buffer's fixed device twin, and replays the graphs.  Buckets are
padded with dummy requests of one token at position 0 whose keys and values go to the cache's
null page.

The captured kernels are the same ones an uncaptured step launches; nothing is compiled or
traced.  A model takes part only if all its parts declare ``graph_safe``.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..csrc import ops
from ..csrc import cdecl as _cdecl
from .batch import LAYOUT_INTS, Entry, next_serial

_K = _cdecl.constants()
HEAD_GRAPH_CALLS = 3          # layer calls in the first of a step's two graphs


class StaticDecodeBatch:
    """The fixed-address twin of `StepBatch` for ``size`` requests of one token each: the same
    sections in one int32 buffer at one device address, refilled for every replay."""

    captured = True             # launches made with it are recorded and replayed with other contents

    def __init__(self, size: int, cache, device, nominal_kv: int):
        B, W, G = size, cache.max_blocks, cache.num_groups
        self.size = size
        self.num_tokens = self.num_seqs = self.num_logit_rows = B
        self.table_width = W
        o_tok, o_pos, o_seq = 0, B, 2 * B
        o_cu = 3 * B
        o_kv = o_cu + B + 1
        o_slot = o_kv + B
        o_rows = o_slot + B
        o_maxkv = o_rows + B
        o_tab = o_maxkv + 1
        total = o_tab + G * B * W
        self._o = (o_tok, o_pos, o_kv, o_slot, o_maxkv, o_tab)
        layout = np.zeros(LAYOUT_INTS, dtype=np.int32)
        for name, v in (("KB_NUM_TOKENS", B), ("KB_NUM_SEQS", B), ("KB_NUM_ROWS", B), ("KB_TABLE_WIDTH", W), ("KB_NUM_GROUPS", G),
                        ("KB_MAX_COUNT", 1), ("KB_MAX_KV_LEN", nominal_kv), ("KB_TOTAL_INTS", total), ("KB_O_TOKEN_IDS", o_tok),
                        ("KB_O_POSITIONS", o_pos), ("KB_O_SEQ_OF_TOKEN", o_seq), ("KB_O_CU_SEQLENS", o_cu), ("KB_O_KV_LENS", o_kv),
                        ("KB_O_SLOTS", o_slot), ("KB_O_ROWS", o_rows), ("KB_O_MAX_KV", o_maxkv), ("KB_O_TABLES", o_tab)):
            layout[_K[name]] = v
        self.layout = layout
        # a ring of pinned buffers: a buffer is rewritten only after the copy that read it is done
        self._ring = [torch.zeros(total, dtype=torch.int32).pin_memory() for _ in range(3)]
        self._ring_np = [t.numpy() for t in self._ring]
        for h in self._ring_np:             # what never changes: request i is token i, and its logits are row i
            h[o_seq:o_seq + B] = np.arange(B)
            h[o_cu:o_cu + B + 1] = np.arange(B + 1)
            h[o_rows:o_rows + B] = np.arange(B)
        self._ring_done = [None, None, None]
        self._turn = 0
        self.host = self._ring_np[0]
        self.serial = next_serial()
        self.dev = torch.zeros(total, dtype=torch.int32, device=device)
        self.device_buffer = self.dev
        self.token_ids = self.dev[o_tok:o_tok + B]
        self.positions = self.dev[o_pos:o_pos + B]
        self.seq_of_token = self.dev[o_seq:o_seq + B]
        self.cu_seqlens = self.dev[o_cu:o_cu + B + 1]
        self.kv_lens = self.dev[o_kv:o_kv + B]
        self.slots = self.dev[o_slot:o_slot + B]
        self.logit_rows = self.dev[o_rows:o_rows + B]
        self._tables = [self.dev[o_tab + g * B * W: o_tab + (g + 1) * B * W].view(B, W) for g in range(G)]
        self.counts = [1] * B
        self.cu_seqlens_host = list(range(B + 1))
        self.slots_host: List[int] = [cache.spare_slot] * B
        self.kv_lens_host: List[int] = [1] * B
        self.max_count = 1
        self.null_page = cache.null_page
        self.spare_slot = cache.spare_slot
        # the context for which a recorded launch plans (the slices of an attention kernel, say);
        # the real longest context is on the device, at KB_O_MAX_KV
        self.max_kv_len = nominal_kv
        self.bytes_h2d = int(total * 4)
        self.fill([], cache)

    @property
    def is_decode_only(self) -> bool:
        return True

    def block_table(self, group: int) -> torch.Tensor:
        return self._tables[group]

    def fill(self, entries: Sequence[Entry], cache) -> None:
        """Writes this step's values into the pinned buffer and starts its copy to the device."""
        o_tok, o_pos, o_kv, o_slot, o_maxkv, o_tab = self._o
        B, W, G = self.size, self.table_width, cache.num_groups
        turn = self._turn
        self._turn = (turn + 1) % len(self._ring)
        if self._ring_done[turn] is not None:
            self._ring_done[turn].synchronize()
        h = self._ring_np[turn]
        n = len(entries)
        max_kv = 1
        if n:
            h[o_tok:o_tok + n] = [e.tokens[0] for e in entries]
            rids = np.fromiter((e.rid for e in entries), dtype=np.int64, count=n)
            max_kv = cache.describe_decode(rids, B, W, h[o_pos:o_pos + B], h[o_kv:o_kv + B], h[o_slot:o_slot + B],
                                           h[o_tab:o_tab + G * B * W])
        if n < B:                       # dummy requests: one token at position 0 on the null page, state in the spare slot
            h[o_tok + n:o_tok + B] = 0
            h[o_pos + n:o_pos + B] = 0
            h[o_kv + n:o_kv + B] = 1
            h[o_slot + n:o_slot + B] = self.spare_slot
            for g in range(G):
                for i in range(n, B):
                    h[o_tab + (g * B + i) * W] = self.null_page
        h[o_maxkv] = max_kv
        self.host = h
        self.serial = next_serial()
        self.slots_host = h[o_slot:o_slot + B].tolist()
        self.kv_lens_host = h[o_kv:o_kv + B].tolist()
        self.dev.copy_(self._ring[turn], non_blocking=True)
        ev = self._ring_done[turn] or torch.cuda.Event()
        ev.record()
        self._ring_done[turn] = ev


class DecodeGraphs:
    """One captured decode step per bucket size, made at first use."""

    def __init__(self, model, cache, batch_max: int):
        self.model, self.cache = model, cache
        self.sizes = []
        s = 1
        while s < batch_max:
            self.sizes.append(s)
            s *= 2
        self.sizes.append(batch_max)
        self._graphs: Dict[tuple, tuple] = {}
        self.launches_per_replay: Dict[tuple, int] = {}

    # A captured launch fixes what its part decided on the host from the context it was recorded
    # for (an attention kernel its number of key-range slices; their length follows the real
    # contexts through device memory).  So that short and very long contexts get decisions that
    # suit them, steps are captured per class of the longest context.
    KV_CLASSES = (1024, 2048, 4096)

    def kv_class(self, max_kv: int) -> int:
        for c in self.KV_CLASSES:
            if max_kv <= c:
                return c
        return max(self.KV_CLASSES[-1] * 2, self.cache.max_blocks * self.cache.page_size)

    def bucket(self, n: int) -> int:
        for s in self.sizes:
            if n <= s:
                return s
        raise ValueError(f"{n} requests exceed the largest bucket {self.sizes[-1]}")

    def _capture(self, size: int, nominal_kv: int):
        dev = self.model.device
        batch = StaticDecodeBatch(size, self.cache, dev, nominal_kv)
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):               # one uncaptured run: loads modules, sets attributes
            self.model.forward(batch, self.cache)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        # Two graphs: the first few layer calls, then the rest.  Submitting a graph of several
        # hundred kernels takes the host longer than a layer takes the GPU; the short first graph
        # is running while the long one is still being submitted.
        n_calls = len(self.model.order)
        head_calls = min(HEAD_GRAPH_CALLS, n_calls // 2)
        first, rest = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        before = ops.launches
        with torch.cuda.graph(first):
            x, pending = self.model.forward_embed(batch)
            x, pending = self.model.forward_calls(x, pending, batch, self.cache, 0, head_calls)
        with torch.cuda.graph(rest, pool=first.pool()):
            x, pending = self.model.forward_calls(x, pending, batch, self.cache, head_calls, n_calls)
            logits = self.model.forward_head(x, pending, batch)
        self.launches_per_replay[(size, nominal_kv)] = ops.launches - before
        self._graphs[(size, nominal_kv)] = ((first, rest), batch, logits)
        return self._graphs[(size, nominal_kv)]

    def capture_all(self, longest_context: int) -> int:
        """Captures every bucket size at every class of context up to ``longest_context`` now, so
        that no step of a later run pays for a capture (a server does this once, at start-up).
        Returns the number of steps captured."""
        classes = sorted({self.kv_class(c) for c in list(self.KV_CLASSES) + [longest_context] if c <= max(longest_context, self.KV_CLASSES[0])}
                         | {self.kv_class(longest_context)})
        made = 0
        for size in self.sizes:
            for nominal in classes:
                if (size, nominal) not in self._graphs:
                    self._capture(size, nominal)
                    made += 1
        return made

    def run(self, entries: Sequence[Entry], token_ids_dev: Optional[torch.Tensor] = None):
        """Replays the bucket's graph for these one-token entries; returns (logits of the
        first len(entries) rows, static batch, kernels replayed).  ``token_ids_dev`` (int32 on the
        device, one id per entry) replaces the entries' token ids: the ids the previous step
        sampled, which the host has not read yet."""
        size = self.bucket(len(entries))
        nominal = self.kv_class(1 + max(self.cache.length(e.rid) for e in entries))
        g = self._graphs.get((size, nominal)) or self._capture(size, nominal)
        graphs, batch, logits = g
        batch.fill(entries, self.cache)
        if token_ids_dev is not None:
            batch.token_ids[:len(entries)].copy_(token_ids_dev[:len(entries)], non_blocking=True)
        for graph in graphs:
            graph.replay()
        return logits[:len(entries)], batch, self.launches_per_replay[(size, nominal)]
