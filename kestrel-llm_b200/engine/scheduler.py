"""Python face of the native scheduler (`csrc/host/scheduler.cpp`).

The scheduler decides, per step: decode tokens of running requests first, then portions of
running prompts under the token budget, then admissions in arrival order; when pages run out
the youngest running request yields and is computed again later.  Token values, sampling
parameters and outputs live in `LLM`; the scheduler sees only counts.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List

from ..cache.manager import PageTable, host_library


class SchedulerError(RuntimeError):
    pass


@dataclass
class Scheduled:
    rid: int
    start: int       # first token of the request that this step runs
    count: int       # how many
    wants_token: bool  # the entry ends with the request's last known token: sample after it


class Scheduler:
    def __init__(self, pages: PageTable, max_step_tokens: int, prefill_chunk: int, batch_max: int,
                 max_queued: int, max_model_len: int):
        self._lib = host_library()
        self._pages = pages
        self._h = self._lib.ksched_create(pages.handle, max_step_tokens, prefill_chunk, batch_max,
                                          min(max_queued, (1 << 31) - 1), max_model_len)
        if not self._h:
            raise SchedulerError("scheduler: bad options")
        cap = batch_max + 8
        self._cap = cap
        self._ids = (ctypes.c_longlong * cap)()
        self._starts = (ctypes.c_int * cap)()
        self._counts = (ctypes.c_int * cap)()
        self._wants = (ctypes.c_int * cap)()

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.ksched_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def add(self, rid: int, prompt_len: int, max_new_tokens: int) -> None:
        rc = self._lib.ksched_add(self._h, rid, prompt_len, max_new_tokens)
        if rc == -1:
            raise SchedulerError(f"request {rid}: the waiting queue is full")
        if rc == -2:
            raise SchedulerError(f"request {rid}: {prompt_len} prompt tokens + {max_new_tokens} new tokens "
                                 f"exceed max_model_len or the whole page pool")
        if rc != 0:
            raise SchedulerError(f"request {rid}: empty prompt or duplicate id")

    def schedule(self) -> List[Scheduled]:
        n = self._lib.ksched_schedule(self._h, self._ids, self._starts, self._counts, self._wants, self._cap)
        if n < 0:
            raise SchedulerError({-7: "schedule() called before the previous step was completed",
                                  -8: "pages vanished between check and reservation"}.get(n, f"scheduler error {n}"))
        return [Scheduled(int(self._ids[i]), int(self._starts[i]), int(self._counts[i]), bool(self._wants[i]))
                for i in range(n)]

    def preempted(self) -> List[int]:
        buf = (ctypes.c_longlong * self._cap)()
        n = self._lib.ksched_preempted(self._h, buf, self._cap)
        return [int(buf[i]) for i in range(min(n, self._cap))]

    def step_done(self) -> None:
        self._lib.ksched_step_done(self._h)

    def on_token(self, rid: int) -> bool:
        """One more token of the request is known.  True if it has reached its token limit."""
        rc = self._lib.ksched_on_token(self._h, rid)
        if rc < 0:
            raise SchedulerError(f"request {rid} is not running")
        return rc == 1

    def finish(self, rid: int) -> None:
        if self._lib.ksched_finish(self._h, rid) != 0:
            raise SchedulerError(f"request {rid} is unknown")

    @property
    def num_running(self) -> int:
        return self._lib.ksched_num_running(self._h)

    @property
    def num_waiting(self) -> int:
        return self._lib.ksched_num_waiting(self._h)

    @property
    def num_preemptions(self) -> int:
        return self._lib.ksched_num_preemptions(self._h)
