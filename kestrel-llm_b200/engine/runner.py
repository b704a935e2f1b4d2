"""Python face of the native step runner (`kestrel_step_raw`, csrc/kernels/step_program.cu).

One call a step: the runner packs the step's description, copies it to the device, and walks
the model's step program, launching every kernel natively.  The host side of a step is then a
few microseconds a kernel instead of an interpreted walk through the parts, which matters for
steps of a few hundred tokens or fewer: their kernels are shorter than such a walk.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import numpy as np
import torch

from ..cache.manager import OutOfPages
from ..csrc import cdecl as _cdecl
from ..csrc import ops
from .batch import Entry, flatten

_K = _cdecl.constants()


class StepRunner:
    def __init__(self, program: ops.StepProgram, cache, max_tokens: int, max_seqs: int, guards: bool = False):
        self._lib = ops.library()
        self.program = program
        self.cache = cache
        self._h = self._lib.krunner_create(program.handle, cache.handle, int(max_tokens), int(max_seqs))
        if not self._h:
            raise ops.KernelError(self._lib.kestrel_last_error().decode("utf-8", "replace"))
        if guards:
            self._lib.krunner_set_guards(self._h, 1)
        self.guards = guards
        self.last_launches = 0
        self.last_h2d_bytes = 0
        self._phase = (ctypes.c_float * ops.PHASE_COUNT)()

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.krunner_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def step(self, entries: Sequence[Entry], vocab: int, profile=None) -> Optional[torch.Tensor]:
        """Runs the entries (pages reserved, requests admitted) and returns float32 logits
        [wanted places, vocab] on the device, or None.  The cache manager is not committed."""
        ids, counts, tokens, want_counts, wants = flatten(entries)
        R = int(wants.shape[0])
        logits = torch.empty((R, vocab), dtype=torch.float32, device=self.cache.device) if R else None
        flags = _K["KSTEP_RESERVED"] | _K["KSTEP_NO_COMMIT"]
        if profile is not None:
            flags |= _K["KSTEP_PROFILE"]
        rc = self._lib.kestrel_step_raw(self._h, len(entries), ids.ctypes.data, counts.ctypes.data, tokens.ctypes.data,
                                        want_counts.ctypes.data, wants.ctypes.data,
                                        logits.data_ptr() if logits is not None else None, vocab, flags, ops._stream())
        if rc == -1:
            raise OutOfPages(self._lib.kestrel_last_error().decode("utf-8", "replace"))
        if rc < 0:
            raise ops.KernelError(self._lib.kestrel_last_error().decode("utf-8", "replace"))
        self.last_launches = rc
        self.last_h2d_bytes = int(self._lib.krunner_last_h2d_bytes(self._h))
        if profile is not None:
            self._lib.krunner_phase_ms(self._h, ctypes.addressof(self._phase))
            profile.add(list(self._phase), int(counts.sum()), int(counts.max()) == 1,
                        seq=max(self.cache.length(int(r)) for r in ids) + int(counts.max()))
        return logits

    @property
    def workspace_bytes(self) -> int:
        return int(self._lib.krunner_workspace_bytes(self._h))

    @property
    def guard_failures(self) -> int:
        return int(self._lib.krunner_guard_failures(self._h))
