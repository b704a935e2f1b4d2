"""Token embedding and the output head.

x = E[token] widened to float32 (st.c:16392-16393); logits = W_lm n in float32
(st.c:16850-16855).  A tied head shares the embedding's memory
(vqf_convert/src/conv_main.c:613-614).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..csrc import ops
from .base import Part, WeightSlot


class TokenEmbedding(Part):
    graph_safe = True

    def __init__(self, vocab: int, width: int, dtype: torch.dtype, device, weight_name: str):
        self.vocab, self.width = vocab, width
        self.weight = torch.empty((vocab, width), dtype=dtype, device=device)
        self.weight_name = weight_name

    def weight_slots(self) -> List[WeightSlot]:
        return [WeightSlot(self.weight_name, self.weight)]

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        out = torch.empty((token_ids.shape[0], self.width), dtype=torch.float32, device=token_ids.device)
        ops.embed(self.weight, token_ids, out)
        return out

    def emit(self, prog) -> int:
        return prog.embed(self.weight)


class LMHead(Part):
    graph_safe = True

    def __init__(self, vocab: int, width: int, dtype: torch.dtype, device, weight_name: str,
                 tied_to: Optional[TokenEmbedding] = None):
        self.vocab, self.width = vocab, width
        self.weight_name = weight_name
        self.tied = tied_to is not None
        self.weight = tied_to.weight if tied_to is not None else \
            torch.empty((vocab, width), dtype=dtype, device=device)

    def weight_slots(self) -> List[WeightSlot]:
        return [] if self.tied else [WeightSlot(self.weight_name, self.weight)]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x [R, width] -> float32 logits [R, vocab].  The product is not split over K (a split
        product returns slices that a consumer kernel sums; the logits have no such consumer)."""
        logits = torch.empty((1, x.shape[0], self.vocab), dtype=torch.float32, device=x.device)
        return ops.linear(x, self.weight, logits, weights_static=True)[0]

    def emit(self, prog, x: int) -> None:
        prog.logits(x, self.weight)
