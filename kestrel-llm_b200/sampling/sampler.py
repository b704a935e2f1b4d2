"""Picks the next token of every request whose logits a step returned, on the device.

Greedy rows take the first maximum.  Other rows are sampled by one kernel with their own
temperature, top-k, min-p and top-p (meanings: src/core/vllm_transformer.c:357-479 of the
reference).  The uniform number of a draw is a function of (request seed, index of the token
being generated) only - the reference draws from the process-wide, never seeded ``rand()``
(vllm_transformer.c:464) - so a request's output does not depend on what it was batched with
and can be repeated.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from ..csrc import ops
from .params import SamplingParams

_MASK = (1 << 64) - 1


def _mix(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def uniform_for(seed: int, index: int) -> float:
    """Uniform number in (0, 1] for the ``index``-th generated token of a request with ``seed``
    (two rounds of the splitmix64 finaliser; 24 bits, so the value is exact in float32)."""
    z = _mix(_mix(seed & _MASK) ^ (index & _MASK))
    return ((z >> 40) + 1) / float(1 << 24)


class Sampler:
    RING = 4        # pinned buffers for the rows' options; a buffer is reused only after its copy has run

    def __init__(self, device):
        self.device = torch.device(device)
        self._ring: List[torch.Tensor] = []
        self._ring_done: List[object] = []
        self._turn = 0

    def _pinned(self, rows: int) -> np.ndarray:
        """A pinned float32 [5, rows] view whose last copy to the device has completed."""
        if not self._ring or self._ring[0].shape[1] < rows:
            cap = max(64, 1 << (rows - 1).bit_length())
            for ev in self._ring_done:
                if ev is not None:
                    ev.synchronize()
            self._ring = [torch.empty((5, cap), dtype=torch.float32).pin_memory() for _ in range(self.RING)]
            self._ring_done = [None] * self.RING
        t = self._turn
        self._turn = (t + 1) % self.RING
        if self._ring_done[t] is not None:
            self._ring_done[t].synchronize()
        self._current = t
        return self._ring[t].numpy()[:, :rows]

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               indices: Sequence[int], generated: Optional[Sequence[Sequence[int]]] = None) -> torch.Tensor:
        """logits float32 [R, V]; row r belongs to a request with ``params[r]``, ``seeds[r]``,
        generating its ``indices[r]``-th token; ``generated[r]`` are the tokens it has generated so
        far (needed by rows with a repetition penalty, which changes ``logits`` in place).
        Returns int32 [R] on the device."""
        R = logits.shape[0]
        out = torch.empty((R,), dtype=torch.int32, device=self.device)
        if any(p.penalised for p in params):
            if generated is None:
                raise ValueError("a repetition penalty needs the tokens generated so far")
            W = 64
            hist = np.full((R, W), -1, dtype=np.int32)
            counts = np.zeros((R,), dtype=np.int32)
            pen = np.ones((R,), dtype=np.float32)
            for r, (p, g) in enumerate(zip(params, generated)):
                if not p.penalised:
                    continue
                last = list(g[-p.repetition_window:])[::-1]       # most recent first, as the reference walks them
                hist[r, :len(last)] = last
                counts[r] = len(last)
                pen[r] = p.repetition_penalty
            ops.repetition_penalty(logits, torch.from_numpy(hist).to(self.device), torch.from_numpy(counts).to(self.device),
                                   torch.from_numpy(pen).to(self.device))
        if all(p.greedy for p in params):
            ops.argmax(logits, out)
            return out
        host = self._pinned(R) if self.device.type == "cuda" else np.empty((5, R), dtype=np.float32)
        ks = np.empty((R,), dtype=np.int32)
        for r, (p, s, i) in enumerate(zip(params, seeds, indices)):
            host[0, r] = p.temperature if not p.greedy else 0.0
            host[1, r] = p.top_p
            host[2, r] = p.min_p
            host[3, r] = uniform_for(s, i)
            ks[r] = p.top_k
        host[4] = ks.view(np.float32)
        if self.device.type == "cuda":
            dev = torch.empty((5, R), dtype=torch.float32, device=self.device)
            dev.copy_(self._ring[self._current][:, :R], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            self._ring_done[self._current] = ev
        else:
            dev = torch.from_numpy(host).to(self.device)
        ops.sample(logits, dev[0], dev[4].view(torch.int32), dev[1], dev[2], dev[3], out)
        return out
