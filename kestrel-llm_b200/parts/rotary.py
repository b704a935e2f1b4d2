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

from .base import PositionEncoding, Rotation


class RotaryHalf(PositionEncoding):
    graph_safe = True

    pairing = "half"

    def __init__(self, head_dim: int, theta: float, device, rotary_dim: Optional[int] = None, scale: float = 1.0):
        rot = head_dim if rotary_dim is None else rotary_dim
        if rot % 2 or rot <= 0 or rot > head_dim:
            raise ValueError(f"rotary size {rot} must be even and at most the head size {head_dim}")
        self.rotary_dim = rot
        self.theta = float(theta)
        self.scale = float(scale)
        half = rot // 2
        j = np.arange(half, dtype=np.float32)
        inv = (np.float32(1.0) / np.power(np.float32(theta), j / np.float32(half), dtype=np.float32))
        self.inv_freq = torch.from_numpy(inv.astype(np.float32)).to(device)

    def rotary(self) -> Rotation:
        return Rotation(self.inv_freq, self.rotary_dim, self.pairing, self.scale)


class RotaryInterleaved(RotaryHalf):
    """The same angles with adjacent pairing: dimension 2j turns with 2j + 1.  No model of the
    reference uses it on this path (its history notes the pairing as a past fault,
    st.c:16478-16483); checkpoints of other families store their heads this way."""

    pairing = "interleaved"


class NoPositionEncoding(PositionEncoding):
    """A mixer that sees no positions (causality alone orders the tokens)."""
