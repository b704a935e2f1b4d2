"""The cache manager's bookkeeping (native, no GPU): no page is lost, held twice or freed
twice, under random orders of requests; windows give pages back; exhaustion changes nothing."""
import random

import numpy as np
import pytest

from kestrel_llm_b200.cache import CacheError, OutOfPages, PageTable


def test_pages_follow_length():
    pt = PageTable([0], [8], page_size=4, max_requests=3, max_blocks_per_request=8)
    assert pt.admit(10) in (0, 1, 2)
    pt.reserve(10, 5)
    assert pt.block_table(10, 0) == [0, 1] and pt.free_pages(0) == 6
    pt.commit(10, 5)
    pt.reserve(10, 3)                      # positions 5..7 fit the second page
    assert pt.block_table(10, 0) == [0, 1]
    pt.commit(10, 3)
    pt.reserve(10, 1)
    assert pt.block_table(10, 0) == [0, 1, 2] and pt.length(10) == 8
    pt.check()
    pt.release(10)
    assert pt.free_pages(0) == 8 and pt.live_requests() == 0
    pt.check()


def test_describe_decode_matches_the_single_queries():
    """The one-call description of a decode step (positions, lengths, slots, block tables of
    every group) agrees with the per-request queries; an unknown request is named."""
    pt = PageTable([0, 6], [12, 12], page_size=4, max_requests=4, max_blocks_per_request=5)
    for rid, n in ((7, 9), (3, 1), (11, 14)):
        pt.admit(rid); pt.reserve(rid, n); pt.commit(rid, n); pt.reserve(rid, 1)
    rids = np.array([11, 7, 3], dtype=np.int64)
    B, W = 4, 5
    pos, kv, slot = (np.full(B, -7, dtype=np.int32) for _ in range(3))
    tables = np.full((2, B, W), -7, dtype=np.int32)
    longest = pt.describe_decode(rids, B, W, pos, kv, slot, tables)
    assert longest == 15
    for i, rid in enumerate(rids.tolist()):
        assert pos[i] == pt.length(rid) and kv[i] == pt.length(rid) + 1 and slot[i] == pt.slot(rid)
        for g in range(2):
            want = pt.block_table(rid, g)
            assert tables[g, i, :len(want)].tolist() == want and (tables[g, i, len(want):] == -1).all()
    assert pos[3] == -7 and (tables[:, 3] == -7).all()          # rows beyond the requests are left alone
    with pytest.raises(CacheError):
        pt.describe_decode(np.array([7, 99], dtype=np.int64), B, W, pos, kv, slot, tables)


def test_freed_pages_are_used_again_first():
    pt = PageTable([0], [6], 4, 4, 6)
    pt.admit(1); pt.reserve(1, 8); pt.commit(1, 8)
    pt.admit(2); pt.reserve(2, 4); pt.commit(2, 4)
    held = pt.block_table(1, 0)
    pt.release(1)
    pt.admit(3); pt.reserve(3, 8)
    assert pt.block_table(3, 0) == held            # the pages just given back, first block first
    pt.check()


def test_exhaustion_changes_nothing():
    pt = PageTable([0], [4], 4, 4, 16)
    pt.admit(1); pt.reserve(1, 12); pt.commit(1, 12)
    pt.admit(2)
    assert not pt.can_reserve(2, 5)
    with pytest.raises(OutOfPages):
        pt.reserve(2, 5)
    assert pt.free_pages(0) == 1 and pt.block_table(2, 0) == []
    pt.reserve(2, 4)
    pt.check()


def test_misuse_is_refused():
    pt = PageTable([0], [4], 4, 2, 2)
    pt.admit(1)
    with pytest.raises(CacheError, match="live already"):
        pt.admit(1)
    pt.admit(2)
    with pytest.raises(CacheError, match="slot"):
        pt.admit(3)
    with pytest.raises(CacheError, match="not live"):
        pt.reserve(9, 1)
    with pytest.raises(CacheError, match="beyond what was reserved"):
        pt.commit(1, 1)
    with pytest.raises(CacheError, match="longest request"):
        pt.reserve(1, 9)
    pt.release(1)
    with pytest.raises(CacheError, match="not live"):
        pt.release(1)                                # freed twice
    pt.check()


def test_window_gives_pages_back():
    # group 0 keeps everything, group 1 the last 6 keys
    pt = PageTable([0, 6], [16, 16], 4, 2, 16)
    pt.admit(1)
    for _ in range(40):
        pt.reserve(1, 1)
        pt.commit(1, 1)
        pt.check()
        L = pt.length(1)
        t = pt.block_table(1, 1)
        lo = max(0, L - 6 + 1)                       # oldest key the next query reaches
        for b, page in enumerate(t):
            if (b + 1) * 4 - 1 < lo:
                assert page == -1, f"block {b} is out of reach at length {L} but still held"
            else:
                assert page >= 0
        assert all(p >= 0 for p in pt.block_table(1, 0))
    assert pt.free_pages(1) >= 16 - 3 and pt.free_pages(0) == 16 - 10
    pt.release(1)
    # a long portion needs every page while it runs (its first query looks at position 0) and
    # gives back all but the window's when it is committed
    pt.admit(2)
    pt.reserve(2, 30)
    assert all(p >= 0 for p in pt.block_table(2, 1)) and pt.free_pages(1) == 16 - 8
    pt.commit(2, 30)
    assert pt.block_table(2, 1)[:6] == [-1] * 6 and pt.free_pages(1) == 16 - 2
    # the next portion starts behind the window's edge: blocks out of reach are never allocated
    pt.reserve(2, 1); pt.commit(2, 1)
    pt.release(2)
    assert pt.free_pages(0) == 16 and pt.free_pages(1) == 16
    pt.check()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders(seed):
    rng = random.Random(seed)
    windows = [0, rng.choice([5, 9, 16])]
    pages = [rng.randint(10, 40), rng.randint(10, 40)]
    ps = rng.choice([1, 4, 16])
    pt = PageTable(windows, pages, ps, max_requests=5, max_blocks_per_request=64)
    live = {}
    next_id = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            pt.admit(next_id); live[next_id] = 0; next_id += 1
        elif op < 0.8 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 7, 20])
            if live[rid] + n > 64 * ps:
                continue
            before = [pt.free_pages(g) for g in range(2)]
            tables = [pt.block_table(rid, g) for g in range(2)]
            if pt.can_reserve(rid, n):
                pt.reserve(rid, n)
                if rng.random() < 0.9:
                    pt.commit(rid, n); live[rid] += n
            else:
                with pytest.raises(OutOfPages):
                    pt.reserve(rid, n)
                assert before == [pt.free_pages(g) for g in range(2)]
                assert tables == [pt.block_table(rid, g) for g in range(2)]
        elif live:
            rid = rng.choice(list(live))
            pt.release(rid); del live[rid]
        pt.check()
        for rid, L in live.items():
            assert pt.length(rid) == L
            t0 = pt.block_table(rid, 0)
            assert len(t0) >= (L + ps - 1) // ps and all(p >= 0 for p in t0)
    for rid in list(live):
        pt.release(rid)
    pt.check()
    assert [pt.free_pages(g) for g in range(2)] == pages and pt.free_slots() == 5
    assert pt.pages_handed_out() > 0
