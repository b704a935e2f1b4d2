"""Pre-norm residual block: x += mixer(norm1(x)); x += ffn(norm2(x))
(reference: st.c:16412-16413 and 16622-16626 for the attention half, st.c:16704-16705 and
16796-16797 for the feed-forward half).  The output of the feed-forward is handed on unadded,
so that the next block's first norm (or the final norm) adds it while normalising - unless the
part added it to the stream itself (a many-token product does that in its epilogue), in which
case nothing is pending.
"""
from __future__ import annotations

import inspect
from typing import List

import torch

from .base import Block, FeedForward, Mixer, Norm, WeightSlot


class PreNormBlock(Block):
    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm, ffn: FeedForward, dtype: torch.dtype):
        self.norm1, self.mixer, self.norm2, self.ffn = norm1, mixer, norm2, ffn
        self.dtype = dtype
        # parts whose forward takes ``residual`` may add their result to the stream themselves
        self._mixer_adds = "residual" in inspect.signature(mixer.forward).parameters
        self._ffn_adds = "residual" in inspect.signature(ffn.forward).parameters

    def parts(self):
        return [self.norm1, self.mixer, self.norm2, self.ffn]

    def weight_slots(self) -> List[WeightSlot]:
        return (self.norm1.weight_slots() + self.mixer.weight_slots() + self.norm2.weight_slots()
                + self.ffn.weight_slots())

    def forward(self, residual: torch.Tensor, pending, batch, cache):
        n = self.norm1.add_forward(residual, pending, self.dtype)
        a = self.mixer.forward(n, batch, cache, residual=residual) if self._mixer_adds else self.mixer.forward(n, batch, cache)
        n = self.norm2.add_forward(residual, a, self.dtype)            # a is None if the mixer added itself
        f = self.ffn.forward(n, batch, residual=residual) if self._ffn_adds else self.ffn.forward(n, batch)
        return residual, f

    @property
    def emits(self) -> bool:
        return all(getattr(p, "emit", None) is not None for p in self.parts())

    def emit(self, prog, residual: int, pending, cache) -> int:
        """This block's operations in a step program; returns the register of what is still to be
        added to the residual stream (the feed-forward's product)."""
        n = self.norm1.emit(prog, residual, pending, self.dtype)
        a = self.mixer.emit(prog, n, residual if self._mixer_adds else None, cache)
        n = self.norm2.emit(prog, residual, a, self.dtype)
        return self.ffn.emit(prog, n, residual if self._ffn_adds else None)
