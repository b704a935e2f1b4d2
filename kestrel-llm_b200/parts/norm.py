"""RMSNorm over the model width, fused with the residual add that precedes it.

out = (x * 1/sqrt(mean(x^2) + eps)) * w with the sum and the scaling in float32
(reference: st.c:8811-8827).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..csrc import ops
from .base import Norm, WeightSlot


class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, width: int, eps: float, device, weight_name: str):
        self.width = width
        self.eps = float(eps)
        self.weight = torch.empty((width,), dtype=torch.float32, device=device)
        self.weight_name = weight_name

    def weight_slots(self) -> List[WeightSlot]:
        return [WeightSlot(self.weight_name, self.weight, "norm")]

    def add_forward(self, residual: torch.Tensor, delta, out_dtype: torch.dtype,
                    rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = residual.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, self.width), dtype=out_dtype, device=residual.device)
        ops.add_rmsnorm(residual, delta, self.weight, self.eps, out, rows=rows)
        return out

    def emit(self, prog, residual: int, delta: Optional[int], out_dtype: torch.dtype, logit_rows: bool = False) -> int:
        return prog.add_rmsnorm(residual, delta, self.weight, self.eps, out_dtype, logit_rows=logit_rows)
