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
    # the reference's streaming harness (src/main.c:3741-3782, VLLM_STREAM_REPPEN / VLLM_STREAM_REPWIN):
    repetition_penalty: float = 1.0   # > 1: logit l of each of the last generated tokens becomes l / p (l >= 0) or l * p
    repetition_window: int = 32       # how many of the last generated tokens (1..64), once per occurrence
    max_tokens: int = 64          # tokens to generate (the reference's API default)
    seed: Optional[int] = None    # None: derived from the engine's seed and the request's number
    stop_token_ids: Tuple[int, ...] = ()
    ignore_eos: bool = False

    def __post_init__(self):
        if not 1 <= int(self.repetition_window) <= 64:
            raise ValueError(f"repetition_window {self.repetition_window} outside 1..64")
        if self.repetition_penalty >= 1e3:
            raise ValueError(f"repetition_penalty {self.repetition_penalty} is not below 1000")

    @property
    def penalised(self) -> bool:
        return self.repetition_penalty > 1.0

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0 or self.top_p <= 0.0
