"""Causal grouped-query attention over the paged cache.

q, k, v = W{q,k,v} x (+bias) in one fused product; optional per-head RMSNorm of q and k
(st.c:9541-9561); rotation (st.c:8950-8991); K and V written to the request's pages; each
query attends to the keys of its request up to itself, or to the last ``window`` of them;
kv head of query head h is (h * kv_heads) / heads (st.c:10782); scale 1/sqrt(head_dim)
(st.c:16549); output projection (st.c:16622-16626).  With ``reads_cache_only`` the layer
writes nothing and attends over a cache that an earlier layer of the same step filled.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from ..csrc import ops
from .base import Mixer, PagedKVSpec, PositionEncoding, WeightSlot
from .linear import Linear


class GroupedQueryAttention(Mixer):

    def __init__(self, width: int, heads: int, kv_heads: int, head_dim: int, dtype: torch.dtype,
                 device, prefix: str, position: Optional[PositionEncoding], qk_norm_eps: Optional[float],
                 bias: bool = False, window: int = 0, planner: Optional[ops.AttentionPlanner] = None):
        if heads % kv_heads:
            raise ValueError(f"{heads} query heads are not a multiple of {kv_heads} kv heads")
        if head_dim % 2 or head_dim > 256:
            raise ValueError(f"head size {head_dim}: the attention kernels take even sizes up to 256")
        self.width, self.heads, self.kv_heads, self.head_dim = width, heads, kv_heads, head_dim
        self.window = int(window)
        self.prefix = prefix
        self.position = position
        self.dtype = dtype
        q, kv = heads * head_dim, kv_heads * head_dim
        self.qkv = Linear(width, q + 2 * kv, dtype, device, bias=bias)
        self.out = Linear(q, width, dtype, device, bias=bias)
        self.qk_norm_eps = qk_norm_eps
        if qk_norm_eps is not None:
            self.q_norm = torch.empty((head_dim,), dtype=torch.float32, device=device)
            self.k_norm = torch.empty((head_dim,), dtype=torch.float32, device=device)
        else:
            self.q_norm = self.k_norm = None
        self.scale = 1.0 / math.sqrt(head_dim)
        # What the attention kernels keep from layer to layer of a step (tile lists, slice
        # scratch).  The layers of a model share one; a layer built alone gets its own.
        self.planner = planner
        if planner is None and dtype == torch.bfloat16 and torch.device(device).type == "cuda":
            self.planner = ops.AttentionPlanner()
        # a recorded decode step needs every request's rows (token, head) to fit one tile of the decode kernels
        self.graph_safe = heads // kv_heads <= 16

    def cache_spec(self) -> PagedKVSpec:
        return PagedKVSpec(self.kv_heads, self.head_dim, self.window)

    def weight_slots(self) -> List[WeightSlot]:
        p = self.prefix
        q, kv = self.heads * self.head_dim, self.kv_heads * self.head_dim
        w = self.qkv.weight
        slots = [WeightSlot(p + "q_proj.weight", w[:q]), WeightSlot(p + "k_proj.weight", w[q:q + kv]),
                 WeightSlot(p + "v_proj.weight", w[q + kv:]), WeightSlot(p + "o_proj.weight", self.out.weight)]
        if self.qkv.bias is not None:
            b = self.qkv.bias
            slots += [WeightSlot(p + "q_proj.bias", b[:q], "bias"), WeightSlot(p + "k_proj.bias", b[q:q + kv], "bias"),
                      WeightSlot(p + "v_proj.bias", b[q + kv:], "bias"), WeightSlot(p + "o_proj.bias", self.out.bias, "bias")]
        if self.q_norm is not None:
            slots += [WeightSlot(p + "q_norm.weight", self.q_norm, "norm"),
                      WeightSlot(p + "k_norm.weight", self.k_norm, "norm")]
        return slots

    def forward(self, x: torch.Tensor, batch, cache, residual: Optional[torch.Tensor] = None) -> Optional[ops.Partials]:
        T = x.shape[0]
        q = torch.empty((T, self.heads * self.head_dim), dtype=self.dtype, device=x.device)
        rot = self.position.rotary() if self.position is not None else None
        table = batch.block_table(cache.group)
        prepare = dict(q_norm_w=self.q_norm, k_norm_w=self.k_norm, norm_eps=self.qk_norm_eps or 0.0,
                       inv_freq=rot.inv_freq if rot else None, rotary_dim=rot.dim if rot else 0, positions=batch.positions,
                       seq_of_token=batch.seq_of_token, block_table=table, page_size=cache.page_size, k_cache=cache.k,
                       v_cache=cache.v, q_out=q, nq=self.heads, nkv=self.kv_heads, hd=self.head_dim, write_kv=cache.writable,
                       rot_mode=rot.mode if rot else 0, rot_scale=rot.scale if rot else 1.0)
        # many tokens of head size 128: one kernel for the product and everything up to attention
        if not ops.qkv_prepare_fused(x, self.qkv.weight, self.qkv.bias, **prepare):
            ops.attn_prepare(self.qkv.forward(x), **prepare)
        a = torch.empty_like(q)
        ops.attention(self.planner, q, cache.k, cache.v, batch, cache.group, cache.page_size, a, self.heads, self.kv_heads,
                      self.head_dim, self.window, self.scale)
        return self.out.forward(a, residual=residual)

    def emit(self, prog, x: int, residual: Optional[int], cache) -> int:
        qkv = self.qkv.emit(prog, x, phase="qkv")
        rot = self.position.rotary() if self.position is not None else None
        q = prog.attn_prepare(qkv, self.q_norm, self.k_norm, self.qk_norm_eps or 0.0, rot.inv_freq if rot else None,
                              rot.dim if rot else 0, rot.mode if rot else 0, rot.scale if rot else 1.0, cache.group,
                              cache.page_size, cache.k, cache.v, self.heads, self.kv_heads, self.head_dim, cache.writable)
        a = prog.attention(q, self.planner, cache.group, cache.page_size, cache.k, cache.v, self.heads, self.kv_heads,
                           self.head_dim, self.window, self.scale)
        return self.out.emit(prog, a, residual=residual, phase="o")
