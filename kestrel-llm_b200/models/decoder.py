"""A decoder as data: an embedding, a list of blocks, the order in which they run, a final
norm and an output head.

``order`` is a list of `LayerCall`s.  A call names the block it runs and the cache layer it
uses; a block may appear in several calls (its weights run twice, each call with a cache
layer of its own or a shared one), and a call with ``writes_cache=False`` reads a cache layer
that an earlier call of the same step filled.  The reference runs its layers in a fixed loop
(src/model/vllm_safetensors.c:16404-16812); here the loop walks this list.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from ..parts.base import Block, CacheSpec, Norm, Part, PositionEncoding, WeightSlot
from ..parts.embedding import LMHead, TokenEmbedding


@dataclass(frozen=True)
class LayerCall:
    block: int                  # index into DecoderModel.blocks
    cache: int = -1             # cache layer it uses, -1 for none
    writes_cache: bool = True   # False: attends over what an earlier call wrote


class DecoderModel(Part):
    def __init__(self, config, dtype: torch.dtype, device, embedding: TokenEmbedding,
                 position: Optional[PositionEncoding], blocks: Sequence[Block],
                 order: Sequence[LayerCall], final_norm: Norm, lm_head: LMHead,
                 optional_tensors: Sequence[str] = ()):
        self.config = config
        self.dtype = dtype
        self.device = torch.device(device)
        self.embedding = embedding
        self.position = position
        self.blocks = list(blocks)
        self.order = list(order)
        self.final_norm = final_norm
        self.lm_head = lm_head
        self.optional_tensors = tuple(optional_tensors)   # may be in a checkpoint, are not used
        n_cache = 1 + max([c.cache for c in self.order], default=-1)
        owners: List[Optional[int]] = [None] * n_cache
        for c in self.order:
            if c.cache >= 0 and c.writes_cache:
                if owners[c.cache] is not None:
                    raise ValueError(f"cache layer {c.cache} is written by two layer calls")
                owners[c.cache] = c.block
        for c in self.order:
            if c.cache >= 0 and not c.writes_cache and owners[c.cache] is None:
                raise ValueError(f"cache layer {c.cache} is read but never written")
        seen = set()
        for c in self.order:        # a reader must come after the writer
            if c.cache >= 0:
                if c.writes_cache:
                    seen.add(c.cache)
                elif c.cache not in seen:
                    raise ValueError(f"cache layer {c.cache} is read before it is written")
        self._cache_owner = owners

    @property
    def graph_safe(self) -> bool:
        """Whether a decode step through the whole model can be captured in a CUDA graph."""
        pos_ok = self.position is None or (getattr(self.position, "graph_safe", False)
                                           or type(self.position).add_to_embedding is PositionEncoding.add_to_embedding)
        return (pos_ok and all(b.graph_safe for b in self.blocks) and self.final_norm.graph_safe
                and self.embedding.graph_safe and self.lm_head.graph_safe)

    @property
    def vocab_size(self) -> int:
        return self.lm_head.vocab

    def cache_specs(self) -> List[CacheSpec]:
        """What each cache layer keeps, taken from the block that writes it."""
        return [self.blocks[b].cache_spec() if b is not None else None for b in self._cache_owner]

    def weight_slots(self) -> List[WeightSlot]:
        slots = self.embedding.weight_slots()
        if self.position is not None:
            slots += self.position.weight_slots()
        for b in self.blocks:
            slots += b.weight_slots()
        slots += self.final_norm.weight_slots() + self.lm_head.weight_slots()
        return slots

    def step_program(self, cache):
        """The whole step as a `StepProgram` for the native runner, or None if some part of the
        model has no ``emit`` (it then runs by the walk below).  ``cache`` is the `CacheManager`
        whose layers the program's attention operations point into."""
        from ..csrc import ops
        pos_ok = self.position is None or type(self.position).add_to_embedding is PositionEncoding.add_to_embedding
        blocks_ok = all(getattr(b, "emit", None) is not None and getattr(b, "emits", False) for b in self.blocks)
        if not (pos_ok and blocks_ok and all(getattr(p, "emit", None) is not None
                                              for p in (self.embedding, self.final_norm, self.lm_head))):
            return None
        prog = ops.StepProgram(self.dtype)
        x = self.embedding.emit(prog)
        pending = None
        for call in self.order:
            lc = cache.layer(call.cache, call.writes_cache) if call.cache >= 0 else None
            prog.begin_call()
            pending = self.blocks[call.block].emit(prog, x, pending, lc)
        prog.begin_call()
        n = self.final_norm.emit(prog, x, pending, self.dtype, logit_rows=True)
        self.lm_head.emit(prog, n)
        return prog

    def forward(self, batch, cache) -> Optional[torch.Tensor]:
        """Runs this step's tokens through every layer call; returns float32 logits
        [len(batch.logit_rows), vocab], or None if no logits are wanted."""
        x, pending = self.forward_embed(batch)
        x, pending = self.forward_calls(x, pending, batch, cache, 0, len(self.order))
        return self.forward_head(x, pending, batch)

    # The three stages of `forward`, for callers that run a step in pieces (a captured decode
    # step is two graphs, so that the second is submitted while the first already runs).
    def forward_embed(self, batch):
        x = self.embedding.forward(batch.token_ids)
        if self.position is not None:
            self.position.add_to_embedding(x, batch)
        return x, None

    def forward_calls(self, x, pending, batch, cache, lo: int, hi: int):
        """Layer calls order[lo:hi] on the residual stream ``x`` and the not yet added ``pending``."""
        for call in self.order[lo:hi]:
            lc = cache.layer(call.cache, call.writes_cache) if call.cache >= 0 else None
            x, pending = self.blocks[call.block].forward(x, pending, batch, lc)
        return x, pending

    def forward_head(self, x, pending, batch) -> Optional[torch.Tensor]:
        if batch.num_logit_rows == 0:
            return None
        n = self.final_norm.add_forward(x, pending, self.dtype, rows=batch.logit_rows)
        return self.lm_head.forward(n)
