"""Rotary position encoding with rotate-half pairing.

half = rot/2; f_j = 1/theta^(j/half); angle = (float)pos * f_j; dimension j pairs with
j + half (reference: st.c:8937-8948 for the frequencies, st.c:8963-8989 for the pairing).  The
frequencies are made once on the host in float32 and kept on the device; angles, cos and sin
are computed in float32 inside the kernel that rotates (`ops.attn_prepare`).  ``rotary_dim``
below the head size rotates only the first dimensions of a head; Qwen3 rotates all.
"""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np
import torch

from .base import PositionEncoding


class RotaryHalf(PositionEncoding):
    graph_safe = True

    def __init__(self, head_dim: int, theta: float, device, rotary_dim: Optional[int] = None):
        rot = head_dim if rotary_dim is None else rotary_dim
        if rot % 2 or rot <= 0 or rot > head_dim:
            raise ValueError(f"rotary size {rot} must be even and at most the head size {head_dim}")
        self.rotary_dim = rot
        self.theta = float(theta)
        half = rot // 2
        j = np.arange(half, dtype=np.float32)
        inv = (np.float32(1.0) / np.power(np.float32(theta), j / np.float32(half), dtype=np.float32))
        self.inv_freq = torch.from_numpy(inv.astype(np.float32)).to(device)

    def rotary(self) -> Tuple[torch.Tensor, int]:
        return self.inv_freq, self.rotary_dim


class NoPositionEncoding(PositionEncoding):
    """A mixer that sees no positions (causality alone orders the tokens)."""
