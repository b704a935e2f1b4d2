"""Gated feed-forward: y = W_down (silu(W_gate x) * W_up x), silu(z) = z / (1 + exp(-z))
(reference: st.c:8904-8914, st.c:3605-3607).  Gate and up are one fused product.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..csrc import ops
from .base import FeedForward, WeightSlot
from .linear import Linear


class GatedMLP(FeedForward):
    graph_safe = True

    def __init__(self, width: int, intermediate: int, dtype: torch.dtype, device, prefix: str,
                 activation: str = "silu"):
        if activation != "silu":
            raise ValueError(f"activation '{activation}' has no kernel; only 'silu'")
        self.width, self.intermediate = width, intermediate
        self.prefix = prefix
        self.dtype = dtype
        self.gate_up = Linear(width, 2 * intermediate, dtype, device)
        self.down = Linear(intermediate, width, dtype, device)

    def weight_slots(self) -> List[WeightSlot]:
        p, ff = self.prefix, self.intermediate
        return [WeightSlot(p + "gate_proj.weight", self.gate_up.weight[:ff]),
                WeightSlot(p + "up_proj.weight", self.gate_up.weight[ff:]),
                WeightSlot(p + "down_proj.weight", self.down.weight)]

    def forward(self, x: torch.Tensor, batch, residual: Optional[torch.Tensor] = None) -> Optional[ops.Partials]:
        act = ops.gate_up_swiglu(x, self.gate_up.weight, self.intermediate, weights_static=True)
        return self.down.forward(act, residual=residual)

    def emit(self, prog, x: int, residual: Optional[int]) -> int:
        act = prog.gate_up_swiglu(x, self.gate_up.weight, self.intermediate)
        return self.down.emit(prog, act, residual=residual, phase="down")
