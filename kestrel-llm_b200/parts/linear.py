"""A weight matrix [out, in] and the product with it, y = x W^T (st.c:8880-8892 of the
reference: weights are used in checkpoint layout, without transposing).

The kernel is chosen by dtype and size: float32 always runs the CUDA-core product with
ascending-k FMA accumulation (the true 32-bit path); bfloat16 runs the tcgen05 tensor-core
product when the sizes fit its tiling rules and the CUDA-core product otherwise.  A part's
weights are loaded once, before any step runs, and the product is told so (``weights_static``):
it may fetch weight tiles while the kernel in front of it still runs.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from .base import Part


class Linear(Part):
    def __init__(self, in_features: int, out_features: int, dtype: torch.dtype, device,
                 bias: bool = False):
        self.in_features = in_features
        self.out_features = out_features
        self.weight = torch.empty((out_features, in_features), dtype=dtype, device=device)
        self.bias = torch.empty((out_features,), dtype=torch.float32, device=device) if bias else None

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None,
                residual: Optional[torch.Tensor] = None) -> Optional[ops.Partials]:
        """x [T, in] in the weight's dtype -> Partials [S, T, out].  With ``residual`` (float32
        [T, out]) the product may add itself to it in its epilogue; it then returns None."""
        if residual is not None and self.bias is None and out is None and ops.linear_add_into(x, self.weight, residual):
            return None
        return ops.Partials(ops.linear(x, self.weight, out, weights_static=True), self.bias)

    def emit(self, prog, x: int, residual: Optional[int] = None, phase: str = "other") -> int:
        """The same product in a step program: register of float32 slices (empty if the product
        added itself to ``residual``)."""
        return prog.linear(x, self.weight, self.bias, add_to=residual, phase=phase)
