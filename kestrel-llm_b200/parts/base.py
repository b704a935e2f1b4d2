"""What a layer is built from, and what each kind of part must offer.

A model is a list of blocks and a list that says in which order they run.  A block arranges a
mixer, a feed-forward and norms around the residual stream; a mixer may use a position
encoding.  Every part takes its sizes and constants as constructor arguments, allocates its
own weights on the device it is given, names the checkpoint tensors that fill them
(`weight_slots`), and says what it needs from the cache (`cache_spec`).  No part knows which
model it is in; a model is assembled layer by layer from a configuration.

Activations: the residual stream is float32 [T, width].  A norm turns it into the storage
dtype (bfloat16 or float32).  A mixer or feed-forward takes that and returns `Partials`
(float32 slices of a projection's output, still to be summed), which the next norm adds to
the residual stream in the same kernel that normalises it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple, Union

import torch


@dataclass
class WeightSlot:
    """One checkpoint tensor and the device memory it fills.

    ``dest`` may be a slice of a larger fused tensor (rows of a fused QKV matrix).  ``init`` is
    the distribution used by the random-weights mode: "linear" N(0, 0.02), "norm"
    1 + N(0, 0.02), "bias" N(0, 0.02)."""
    name: str
    dest: torch.Tensor
    init: str = "linear"


@dataclass(frozen=True)
class PagedKVSpec:
    """Keys and values of every token, or of the last ``window`` tokens, in pages."""
    kv_heads: int
    head_dim: int
    window: int = 0          # 0 = all keys


@dataclass(frozen=True)
class FixedStateSpec:
    """A region of constant size per live request (recurrent state and the like)."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


CacheSpec = Union[PagedKVSpec, FixedStateSpec, None]


class Part:
    """Base of all parts: weights by checkpoint name.

    ``graph_safe`` says that ``forward`` only launches kernels whose arguments are device
    tensors of the batch (no value of the batch is read on the host), so a decode step through
    the part can be captured in a CUDA graph and replayed with other contents.  The default is
    False; the engine captures only if every part of the model says True."""

    graph_safe = False

    def weight_slots(self) -> List[WeightSlot]:
        return []

    # A part may also offer ``emit``: it writes the kernel-level operations of its forward pass
    # into a `StepProgram` (csrc/ops.py), once, when the engine is made, and returns the
    # program's register of its result.  The operations must be the ones ``forward`` launches,
    # in the same order.  If every part of a model offers it, steps run from that program through
    # the native runner (one call a step); otherwise they walk the parts' ``forward``.  The
    # signatures mirror ``forward`` with registers in place of tensors:
    #   Norm.emit(prog, residual, delta, out_dtype, logit_rows=False) -> register
    #   Mixer.emit(prog, x, residual, layer_cache) -> register of a product, still to be added
    #   FeedForward.emit(prog, x, residual) -> register of a product
    #   Block.emit(prog, residual, pending, layer_cache) -> pending register
    emit = None


@dataclass(frozen=True)
class Rotation:
    """How a mixer turns queries and keys by position: pair j of the first ``dim`` dimensions of a
    head is turned by the angle position * inv_freq[j].  ``pairing`` "half" pairs dimension j
    with j + dim/2 (the reference's, st.c:8963-8989), "interleaved" pairs 2j with 2j + 1;
    ``scale`` multiplies cos and sin (1 for plain rotary encodings)."""
    inv_freq: torch.Tensor      # float32 [dim / 2] on the device
    dim: int
    pairing: str = "half"
    scale: float = 1.0

    @property
    def mode(self) -> int:
        if self.pairing not in ("half", "interleaved"):
            raise ValueError(f"rotation pairing '{self.pairing}' is neither 'half' nor 'interleaved'")
        return 0 if self.pairing == "half" else 1


class PositionEncoding(Part):
    """How positions enter the model.

    ``rotary()`` returns a `Rotation` for mixers that rotate queries and keys, or None.
    ``add_to_embedding(x, batch)`` lets an absolute encoding add to the embedded tokens; the
    default does nothing."""

    def rotary(self) -> Optional[Rotation]:
        return None

    def add_to_embedding(self, x: torch.Tensor, batch) -> None:
        return None


class Norm(Part):
    """``add_forward(residual, delta, out_dtype, rows=None)``: residual += delta (a Partials or
    None), in place unless ``rows`` selects a subset; returns norm(residual) in out_dtype."""

    def add_forward(self, residual: torch.Tensor, delta, out_dtype: torch.dtype,
                    rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class Mixer(Part):
    """Mixes information between the tokens of a request (attention, recurrence ...).

    ``cache_spec()`` says what it keeps per request.  ``forward(x, batch, cache)`` takes the
    normed activations [T, width] of this step's tokens and the layer's `LayerCache`, reads and
    updates the cache for exactly these tokens, and returns Partials [S, T, width].  A mixer
    whose ``forward`` has a fourth parameter ``residual`` is given the float32 residual stream
    [T, width] and may add its result to it itself (the last product's epilogue); it then returns
    None."""

    def cache_spec(self) -> CacheSpec:
        return None

    def forward(self, x: torch.Tensor, batch, cache):
        raise NotImplementedError


class FeedForward(Part):
    """Token-wise transformation: ``forward(x, batch)`` -> Partials [S, T, width]; with a third
    parameter ``residual`` it may add its result to the residual stream itself and return None,
    as a mixer may."""

    def forward(self, x: torch.Tensor, batch):
        raise NotImplementedError


class Block(Part):
    """Arrangement of parts around the residual stream.

    ``forward(residual, pending, batch, cache)`` -> (residual, pending): ``pending`` is a
    Partials not yet added to the residual stream (the previous block's last output), so that
    the add is fused into the first norm of the next block."""

    mixer: Mixer

    def cache_spec(self) -> CacheSpec:
        return self.mixer.cache_spec()

    @property
    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", False) for p in self.parts())

    def parts(self) -> Sequence[Part]:
        """The parts this block arranges (for checks that concern all of them)."""
        return [self.mixer]

    def forward(self, residual: torch.Tensor, pending, batch, cache):
        raise NotImplementedError
