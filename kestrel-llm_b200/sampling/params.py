"""Sampling options of one request, with the reference's names and meanings
(src/core/vllm_transformer.c:357-479; server defaults src/serve/vllm_server.c:2606-2628).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass
class SamplingParams:
    temperature: float = 0.0      # <= 0: greedy, the first maximum wins
    top_p: float = 1.0            # <= 0: greedy; < 1: shortest most-probable prefix reaching this mass
    top_k: int = 0                # 0 = off
    min_p: float = 0.0            # drop tokens below min_p * the largest probability
    max_tokens: int = 64          # tokens to generate (the reference's API default)
    seed: Optional[int] = None    # None: derived from the engine's seed and the request's number
    stop_token_ids: Tuple[int, ...] = ()
    ignore_eos: bool = False

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0 or self.top_p <= 0.0
