"""Where a step's time goes, by phase, in the reference's own line formats.

The reference accumulates wall-clock time per phase of its decode forward when VLLM_DEC_PROF is
set and prints `[DEC-SINGLE]` lines (src/model/vllm_safetensors.c:16375-16382, 16899-16923),
and prints `[PREFILL-TIMING] ... GEMM/ATTN/OTHER` after every prefill (:18808-18818).  Here
the native runner brackets every operation of a step with CUDA events when asked
(`EngineOptions.profile`), sums them by phase, and this class keeps the sums and prints the same
two lines - device time instead of wall-clock time, milliseconds like the reference.
"""
from __future__ import annotations

import sys
from typing import List

from ..csrc import ops


class PhaseProfile:
    def __init__(self, stream=None):
        self.stream = stream or sys.stderr
        self.decode_ms = [0.0] * ops.PHASE_COUNT
        self.decode_steps = 0
        self.prefill_ms = [0.0] * ops.PHASE_COUNT
        self.prefill_steps = 0
        self.prefill_tokens = 0

    def add(self, phase_ms: List[float], tokens: int, decode_only: bool) -> None:
        """One step's milliseconds per phase (indexed as `ops.PHASES`)."""
        if decode_only:
            self.decode_steps += 1
            for i, v in enumerate(phase_ms):
                self.decode_ms[i] += v
        else:
            self.prefill_steps += 1
            self.prefill_tokens += tokens
            for i, v in enumerate(phase_ms):
                self.prefill_ms[i] += v
            self.print_prefill(phase_ms, tokens)

    def print_prefill(self, ms: List[float], tokens: int) -> None:
        P = ops.PHASES
        gemm = ms[P["qkv"]] + ms[P["o"]] + ms[P["gate_up"]] + ms[P["down"]] + ms[P["lm_head"]]
        attn = ms[P["attn"]]
        total = sum(ms)
        other = total - gemm - attn
        pct = (lambda v: 100.0 * v / total) if total > 0 else (lambda v: 0.0)
        print(f"[PREFILL-TIMING] {tokens} tokens: total={total:.2f}ms  GEMM={gemm:.2f}ms({pct(gemm):.1f}%)  "
              f"ATTN={attn:.2f}ms({pct(attn):.1f}%)  OTHER={other:.2f}ms({pct(other):.1f}%)", file=self.stream, flush=True)

    def print_decode(self) -> None:
        """The decode steps so far, per step, as the reference's `[DEC-SINGLE]` line."""
        if not self.decode_steps:
            return
        P, n = ops.PHASES, self.decode_steps
        m = [v / n for v in self.decode_ms]
        print(f"[DEC-SINGLE] steps={n} per-step ms: qkv={m[P['qkv']]:.3f} attn={m[P['attn']]:.3f} o={m[P['o']]:.3f} "
              f"gu={m[P['gate_up']]:.3f} down={m[P['down']]:.3f} lm={m[P['lm_head']]:.3f} nrm={m[P['norm']]:.3f} "
              f"rope={m[P['rope']]:.3f} emb={m[P['embed']]:.3f} total={sum(m):.3f}", file=self.stream, flush=True)
