"""Where a step's time goes, by phase, in the reference's own line formats.

The reference accumulates wall-clock time per phase of its decode forward when VLLM_DEC_PROF is
set and prints `[DEC-SINGLE]` lines (src/model/vllm_safetensors.c:16375-16382, 16899-16923),
and prints `[PREFILL-TIMING] ... GEMM/ATTN/OTHER` after every prefill (:18808-18818).  Here
the native runner brackets every operation of a step with CUDA events when asked
(`EngineOptions.profile`), sums them by phase, and this class keeps the sums and prints the same
lines - device time instead of wall-clock time, milliseconds like the reference.
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

    def add(self, phase_ms: List[float], tokens: int, decode_only: bool, seq: int = 0) -> None:
        """One step's milliseconds per phase (indexed as `ops.PHASES`); the step's line is printed."""
        if decode_only:
            self.decode_steps += 1
            for i, v in enumerate(phase_ms):
                self.decode_ms[i] += v
            self.print_decode(phase_ms, seq)
        else:
            self.prefill_steps += 1
            self.prefill_tokens += tokens
            for i, v in enumerate(phase_ms):
                self.prefill_ms[i] += v
            self.print_prefill(phase_ms, tokens)

    def print_prefill(self, ms: List[float], tokens: int) -> None:
        """The two lines the reference prints after a prefill (st.c:18808-18831); the output head,
        which the reference times apart, counts under OTHER as there."""
        P = ops.PHASES
        gemm = ms[P["qkv"]] + ms[P["o"]] + ms[P["gate_up"]] + ms[P["down"]]
        attn = ms[P["attn"]]
        total = sum(ms)
        other = total - gemm - attn
        pct = (lambda v: 100.0 * v / total) if total > 0 else (lambda v: 0.0)
        print(f"[PREFILL-TIMING] n={tokens} total={total:.1f}ms | GEMM={gemm:.1f}ms({pct(gemm):4.1f}%) "
              f"ATTN={attn:.1f}ms({pct(attn):4.1f}%) OTHER={other:.1f}ms({pct(other):4.1f}%)", file=self.stream)
        if gemm > 0:
            g = lambda v: 100.0 * v / gemm
            print(f"[PREFILL-KERNELS] QKV={ms[P['qkv']]:.1f}ms({g(ms[P['qkv']]):4.1f}%) O={ms[P['o']]:.1f}ms({g(ms[P['o']]):4.1f}%) "
                  f"GATEUP={ms[P['gate_up']]:.1f}ms({g(ms[P['gate_up']]):4.1f}%) DOWN={ms[P['down']]:.1f}ms({g(ms[P['down']]):4.1f}%)",
                  file=self.stream, flush=True)

    def print_decode(self, ms: List[float], seq: int) -> None:
        """One decode step as the reference's `[DEC-SINGLE]` line (st.c:16913-16919).  The cache
        write is part of the rotation kernel (`rope`) and the activation part of the gate/up
        product (`gu`) here, so `kv` and `silu` are 0; `other` holds the embedding."""
        P = ops.PHASES
        total = sum(ms)
        print(f"[DEC-SINGLE] seq={seq} qkv={ms[P['qkv']]:.2f} attn={ms[P['attn']]:.2f} o={ms[P['o']]:.2f} gu={ms[P['gate_up']]:.2f} "
              f"down={ms[P['down']]:.2f} lm={ms[P['lm_head']]:.2f} nrm={ms[P['norm']]:.2f} rope={ms[P['rope']]:.2f} kv=0.00 silu=0.00 "
              f"othloop=0.00 other={ms[P['embed']] + ms[P['other']]:.2f} total={total:.2f}", file=self.stream, flush=True)

    def mean_decode_ms(self) -> List[float]:
        n = max(1, self.decode_steps)
        return [v / n for v in self.decode_ms]

    def print_summary(self) -> None:
        """Means over the steps seen so far, one line per kind of step."""
        P = ops.PHASES
        if self.decode_steps:
            m = self.mean_decode_ms()
            print(f"[DEC-PROF] {self.decode_steps} decode steps, mean ms: qkv={m[P['qkv']]:.3f} attn={m[P['attn']]:.3f} o={m[P['o']]:.3f} "
                  f"gu={m[P['gate_up']]:.3f} down={m[P['down']]:.3f} lm={m[P['lm_head']]:.3f} nrm={m[P['norm']]:.3f} rope={m[P['rope']]:.3f} "
                  f"total={sum(m):.3f}", file=self.stream, flush=True)
        if self.prefill_steps:
            t = sum(self.prefill_ms)
            print(f"[PREFILL-PROF] {self.prefill_steps} steps with prompt portions, {self.prefill_tokens} tokens, {t:.1f} ms on the device "
                  f"({self.prefill_tokens / max(t, 1e-9) * 1000.0:.0f} tok/s)", file=self.stream, flush=True)
