"""Cache manager: the host-side bookkeeping (native, `csrc/host/cache_manager.cpp`) and the
device memory it describes.

Layers are sorted into groups by what they must keep: all keys, or a window of them.  Each
group has its own pool of pages and its own block table per request; layers of a group share
the table, each with K and V planes of its own laid out [page][kv_head][slot][head_dim].
Beside the pages, every live request owns one slot; layers that keep fixed-size state get a
tensor [slots, *shape] indexed by it.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..csrc import build as _build
from ..csrc import cdecl as _cdecl
from ..parts.base import CacheSpec, FixedStateSpec, PagedKVSpec


class CacheError(RuntimeError):
    pass


class OutOfPages(CacheError):
    pass


_host = None


def host_library() -> ctypes.CDLL:
    """The native host runtime (cache manager and scheduler), built on first use."""
    global _host
    if _host is None:
        # global symbols: the kernel library, loaded later, calls the cache manager of this one
        lib = ctypes.CDLL(_build.build_host(), mode=ctypes.RTLD_GLOBAL)
        _cdecl.declare(lib, ("kcache_", "ksched_", "kbatch_"))
        _host = lib
    return _host


@dataclass(frozen=True)
class GroupInfo:
    window: int              # 0 = all keys
    num_pages: int
    layers: Tuple[int, ...]  # cache layers that share this group's block tables


class LayerCache:
    """What one layer call sees of the cache."""

    __slots__ = ("index", "group", "page_size", "k", "v", "state", "writable", "spec")

    def __init__(self, index, group, page_size, k, v, state, writable, spec):
        self.index, self.group, self.page_size = index, group, page_size
        self.k, self.v, self.state, self.writable, self.spec = k, v, state, writable, spec


class PageTable:
    """The native bookkeeping alone (no device memory): groups, pages, block tables, slots."""

    def __init__(self, windows: Sequence[int], num_pages: Sequence[int], page_size: int,
                 max_requests: int, max_blocks_per_request: int):
        self._lib = host_library()
        n = len(windows)
        W = (ctypes.c_int * max(1, n))(*windows)
        P = (ctypes.c_int * max(1, n))(*num_pages)
        self._h = self._lib.kcache_create(n, ctypes.addressof(W), ctypes.addressof(P), page_size, max_requests,
                                          max_blocks_per_request)
        if not self._h:
            raise CacheError("cache manager: bad sizes")
        self.page_size = page_size
        self.num_groups = n
        self.max_requests = max_requests
        self.max_blocks = max_blocks_per_request

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.kcache_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def handle(self):
        return self._h

    def admit(self, rid: int) -> int:
        slot = self._lib.kcache_admit(self._h, rid)
        if slot == -1:
            raise CacheError(f"no free state slot for request {rid} ({self.max_requests} live)")
        if slot == -2:
            raise CacheError(f"request {rid} is live already")
        return slot

    def can_reserve(self, rid: int, n_new: int) -> bool:
        rc = self._lib.kcache_can_reserve(self._h, rid, n_new)
        if rc < 0:
            raise CacheError(self._explain(rc, rid))
        return rc == 1

    def reserve(self, rid: int, n_new: int) -> None:
        rc = self._lib.kcache_reserve(self._h, rid, n_new)
        if rc == -1:
            raise OutOfPages(f"request {rid}: no pages left for {n_new} more tokens "
                             f"(free per group: {[self.free_pages(g) for g in range(self.num_groups)]})")
        if rc != 0:
            raise CacheError(self._explain(rc, rid))

    def commit(self, rid: int, n_new: int) -> None:
        rc = self._lib.kcache_commit(self._h, rid, n_new)
        if rc != 0:
            raise CacheError(self._explain(rc, rid))

    def release(self, rid: int) -> None:
        rc = self._lib.kcache_release(self._h, rid)
        if rc != 0:
            raise CacheError(self._explain(rc, rid))

    def length(self, rid: int) -> int:
        n = self._lib.kcache_length(self._h, rid)
        if n < 0:
            raise CacheError(self._explain(n, rid))
        return n

    def slot(self, rid: int) -> int:
        s = self._lib.kcache_slot(self._h, rid)
        if s < 0:
            raise CacheError(self._explain(s, rid))
        return s

    def is_live(self, rid: int) -> bool:
        return self._lib.kcache_slot(self._h, rid) >= 0

    def num_blocks(self, rid: int, group: int) -> int:
        return self._lib.kcache_num_blocks(self._h, rid, group)

    def block_table_into(self, rid: int, group: int, row: np.ndarray) -> int:
        """Fill ``row`` (int32, contiguous) with the request's pages, -1 beyond them."""
        return self._lib.kcache_block_table(self._h, rid, group, row.ctypes.data, row.shape[0])

    def describe_decode(self, rids: np.ndarray, batch: int, width: int, pos: np.ndarray, kv: np.ndarray,
                        slot: np.ndarray, tables: np.ndarray) -> int:
        """For a step in which each request of ``rids`` (int64) brings one token: fills positions,
        lengths after the step, slots (int32 views of at least len(rids) entries) and the block
        tables of every group (int32 [groups, batch, width]) in one native call; returns the
        longest length after the step."""
        bad = ctypes.c_int(0)
        rc = self._lib.kcache_describe_decode(self._h, rids.ctypes.data, rids.shape[0], batch, width, pos.ctypes.data,
                                              kv.ctypes.data, slot.ctypes.data, tables.ctypes.data, ctypes.addressof(bad))
        if rc < 0:
            raise CacheError(self._explain(rc, int(rids[bad.value])))
        return rc

    def block_table(self, rid: int, group: int) -> List[int]:
        n = self.num_blocks(rid, group)
        row = np.empty(max(n, 1), dtype=np.int32)
        self.block_table_into(rid, group, row)
        return row[:n].tolist()

    def take_admitted(self) -> List[Tuple[int, int]]:
        """(request, slot) of every admission since the last call, whoever made it (this object's
        `admit` or the native scheduler): the owner of per-slot device state clears those slots."""
        cap = self.max_requests + 8
        ids = (ctypes.c_longlong * cap)()
        slots = (ctypes.c_int * cap)()
        n = self._lib.kcache_take_admitted(self._h, ctypes.addressof(ids), ctypes.addressof(slots), cap)
        return [(int(ids[i]), int(slots[i])) for i in range(min(n, cap))]

    def shuffle_free(self, seed: int = 0) -> None:
        """Free pages in a pseudo-random order fixed by ``seed``: the scattered layout a pool has
        after long serving, from the start (benchmarks, tests)."""
        self._lib.kcache_shuffle_free(self._h, int(seed))

    def free_pages(self, group: int) -> int:
        return self._lib.kcache_free_pages(self._h, group)

    def num_pages(self, group: int) -> int:
        return self._lib.kcache_num_pages(self._h, group)

    def live_requests(self) -> int:
        return self._lib.kcache_live_requests(self._h)

    def free_slots(self) -> int:
        return self._lib.kcache_free_slots(self._h)

    def pages_handed_out(self) -> int:
        return self._lib.kcache_pages_handed_out(self._h)

    def check(self) -> None:
        rc = self._lib.kcache_check(self._h)
        if rc != 0:
            what = {-10: "page id out of range", -11: "page both free and owned", -12: "page free twice",
                    -13: "page held but not marked", -14: "page held twice", -15: "page lost",
                    -16: "slot free twice", -17: "slot held twice", -18: "slot lost"}.get(rc, str(rc))
            raise CacheError(f"cache manager invariant broken: {what}")

    @staticmethod
    def _explain(rc: int, rid: int) -> str:
        return {-3: f"request {rid} is not live", -4: f"request {rid} would exceed the longest request the "
                "block table holds", -5: f"request {rid}: commit beyond what was reserved",
                -6: "no such cache group"}.get(rc, f"cache manager error {rc} for request {rid}")


class CacheManager(PageTable):
    """Bookkeeping plus the device memory of every cache layer.

    ``specs[i]`` is what cache layer i keeps (a `PagedKVSpec`, a `FixedStateSpec` or None).
    ``num_pages`` pages go to every group."""

    def __init__(self, specs: Sequence[CacheSpec], dtype: torch.dtype, device, page_size: int,
                 num_pages: int, max_requests: int, max_model_len: int):
        windows: List[int] = []
        members: List[List[int]] = []
        self.layer_group: List[int] = []
        for i, sp in enumerate(specs):
            if isinstance(sp, PagedKVSpec):
                if sp.window not in windows:
                    windows.append(sp.window)
                    members.append([])
                g = windows.index(sp.window)
                members[g].append(i)
                self.layer_group.append(g)
            else:
                self.layer_group.append(-1)
        max_blocks = (max_model_len + page_size - 1) // page_size
        super().__init__(windows, [num_pages] * len(windows), page_size, max_requests, max_blocks)
        self.groups = [GroupInfo(w, num_pages, tuple(m)) for w, m in zip(windows, members)]
        self.specs = list(specs)
        self.null_page = num_pages
        self.spare_slot = max_requests
        self.dtype, self.device = dtype, torch.device(device)
        self.k: List[Optional[torch.Tensor]] = []
        self.v: List[Optional[torch.Tensor]] = []
        self.state: List[Optional[torch.Tensor]] = []
        for sp in specs:
            if isinstance(sp, PagedKVSpec):
                # one page more than the manager hands out: the "null page", where padding tokens
                # of a captured step write their keys and values
                shape = (num_pages + 1, sp.kv_heads, page_size, sp.head_dim)
                self.k.append(torch.zeros(shape, dtype=dtype, device=device))
                self.v.append(torch.zeros(shape, dtype=dtype, device=device))
                self.state.append(None)
            elif isinstance(sp, FixedStateSpec):
                self.k.append(None)
                self.v.append(None)
                # one slot more than there are requests: the spare slot, which padding rows of a
                # captured step use so that they never touch a live request's state
                self.state.append(torch.zeros((max_requests + 1,) + tuple(sp.shape), dtype=sp.dtype, device=device))
            else:
                self.k.append(None)
                self.v.append(None)
                self.state.append(None)

    def admit(self, rid: int) -> int:
        slot = super().admit(rid)
        self.clear_admitted()
        return slot

    def clear_admitted(self) -> None:
        """A new request starts from zero state: clears the state slot of every request admitted
        since the last call, by `admit` here or by the native scheduler on its own (a slot that a
        finished or preempted request left keeps that request's state until then).  The engine
        calls this before every step."""
        new = self.take_admitted()
        if not new or not any(st is not None for st in self.state):
            return
        for _rid, slot in new:
            for st in self.state:
                if st is not None:
                    st[slot].zero_()

    def layer(self, index: int, writable: bool = True) -> LayerCache:
        return LayerCache(index, self.layer_group[index], self.page_size, self.k[index], self.v[index],
                          self.state[index], writable, self.specs[index])

    def bytes_per_token(self) -> int:
        n = 0
        for sp in self.specs:
            if isinstance(sp, PagedKVSpec):
                n += 2 * sp.kv_heads * sp.head_dim * torch.empty((), dtype=self.dtype).element_size()
        return n
