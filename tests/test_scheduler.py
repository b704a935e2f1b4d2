"""The scheduler's decisions (native, no GPU), driven with a stand-in for the model step."""
import pytest

from kestrel_llm_b200.cache import PageTable
from kestrel_llm_b200.engine.scheduler import Scheduler, SchedulerError


def make(pages=64, page_size=4, budget=32, chunk=16, batch_max=4, max_queued=100, max_len=256, slots=None):
    pt = PageTable([0], [pages], page_size, slots or batch_max, (max_len + page_size - 1) // page_size)
    return pt, Scheduler(pt, budget, chunk, batch_max, max_queued, max_len)


def run_step(pt, s, plan, finish=()):
    """What LLM.step does around the model: commit, count, sample one token where wanted."""
    for e in plan:
        pt.commit(e.rid, e.count)
    s.step_done()
    done = []
    for e in plan:
        if e.wants_token:
            at_limit = s.on_token(e.rid)
            if at_limit or e.rid in finish:
                s.finish(e.rid)
                done.append(e.rid)
    pt.check()
    return done


def test_prompt_is_cut_under_the_budget_and_decodes_go_first():
    pt, s = make(budget=20, chunk=16)
    s.add(1, 40, 4)
    s.add(2, 10, 4)
    p = s.schedule()
    assert [(e.rid, e.start, e.count, e.wants_token) for e in p] == [(1, 0, 16, False), (2, 0, 4, False)]
    run_step(pt, s, p)
    p = s.schedule()                       # oldest first, each at most a chunk, 20 in all
    assert [(e.rid, e.start, e.count, e.wants_token) for e in p] == [(1, 16, 16, False), (2, 4, 4, False)]
    run_step(pt, s, p)
    p = s.schedule()
    assert [(e.rid, e.start, e.count, e.wants_token) for e in p] == [(1, 32, 8, True), (2, 8, 2, True)]
    run_step(pt, s, p)
    s.add(3, 30, 2)
    p = s.schedule()                       # decode tokens first, the new prompt takes the rest
    assert [(e.rid, e.start, e.count, e.wants_token) for e in p] == [(1, 40, 1, True), (2, 10, 1, True), (3, 0, 16, False)]
    run_step(pt, s, p)


def test_finish_by_length_frees_pages_and_slot():
    pt, s = make()
    s.add(7, 5, 2)
    run_step(pt, s, s.schedule())          # prompt, first token
    assert pt.length(7) == 5
    done = run_step(pt, s, s.schedule())   # second token reaches the limit
    assert done == [7] and pt.live_requests() == 0 and pt.free_pages(0) == 64
    assert s.schedule() == [] and s.num_running == 0


def test_admission_limits():
    pt, s = make(batch_max=2, max_queued=2)
    s.add(1, 4, 1); s.add(2, 4, 1)
    with pytest.raises(SchedulerError, match="queue is full"):
        s.add(3, 4, 1)
    p = s.schedule()
    assert {e.rid for e in p} == {1, 2}
    s.add(3, 4, 1)
    run_step(pt, s, p)                     # both sampled their only token and finished
    assert [e.rid for e in s.schedule()] == [3]
    with pytest.raises(SchedulerError, match="exceed"):
        s.add(4, 300, 1)                   # longer than max_model_len
    with pytest.raises(SchedulerError, match="exceed"):
        make(pages=4)[1].add(1, 20, 1)     # longer than the whole pool
    with pytest.raises(SchedulerError, match="empty prompt or duplicate"):
        s.add(3, 4, 1)
    with pytest.raises(SchedulerError, match="before the previous step"):
        s.schedule()


def test_arrival_order_is_kept_when_pages_are_short():
    pt, s = make(pages=8, budget=64, chunk=64)          # 32 tokens in all
    s.add(1, 20, 4)
    s.add(2, 20, 4)                                     # cannot start beside request 1
    s.add(3, 2, 1)                                      # would fit, but must not overtake request 2
    p = s.schedule()
    assert [(e.rid, e.count) for e in p] == [(1, 20)]
    run_step(pt, s, p)
    assert [e.rid for e in s.schedule()] == [1]


def test_pages_run_out_the_youngest_yields_and_is_computed_again():
    pt, s = make(pages=6, page_size=4, budget=64, chunk=64)       # 24 tokens
    s.add(1, 10, 12)
    s.add(2, 9, 12)
    run_step(pt, s, s.schedule())                                 # both prompts: 3 + 3 pages, pool full
    assert pt.free_pages(0) == 0 and s.num_running == 2
    generated = {1: 1, 2: 1}
    for _ in range(2):                                            # lengths 10->12 and 9->11 fit their pages
        p = s.schedule()
        assert sorted(e.rid for e in p) == [1, 2] and s.preempted() == []
        run_step(pt, s, p)
        generated[1] += 1; generated[2] += 1
    p = s.schedule()                                              # request 1 needs a 4th page: 2 yields
    assert s.preempted() == [2] and [e.rid for e in p] == [1]
    assert s.num_waiting == 1 and s.num_preemptions == 1 and not pt.is_live(2)
    run_step(pt, s, p)
    # request 2 comes back with all its tokens, prompt and generated, once pages allow
    while pt.is_live(1):
        p = s.schedule()
        run_step(pt, s, p)
    p = s.schedule()
    assert [(e.rid, e.start, e.count, e.wants_token) for e in p] == [(2, 0, 9 + generated[2], True)]
    pt.check()


def test_stuck_prompts_resolve():
    # two prompts admitted side by side fill the pool before either is complete: the second was
    # admitted while its 20 tokens fitted what was free, but the first still grows
    pt, s = make(pages=8, page_size=4, budget=16, chunk=8)        # 32 tokens
    s.add(1, 28, 2)
    s.add(2, 20, 2)
    seen_preempt = False
    done = []
    for _ in range(40):
        p = s.schedule()
        seen_preempt |= bool(s.preempted())
        if not p:
            break
        done += run_step(pt, s, p)
    assert seen_preempt and done == [1, 2]
    assert pt.free_pages(0) == 8


def test_a_request_is_admitted_only_if_all_its_tokens_fit_now():
    """Admission asks for free pages for everything the request has so far, not for its first
    portion only (it would be preempted a few steps later), and the call that preempts a
    request does not admit it again."""
    pt, s = make(pages=8, page_size=4, budget=16, chunk=8)        # 32 tokens
    s.add(1, 28, 2)
    s.add(2, 28, 2)                                               # its first portion would fit beside request 1, its 28 tokens do not
    p = s.schedule()
    assert [(e.rid, e.count) for e in p] == [(1, 8)] and s.num_waiting == 1
    done = []
    for _ in range(40):
        done += run_step(pt, s, p)
        p = s.schedule()
        assert s.preempted() == []
        if not p:
            break
    assert done == [1, 2] and s.num_preemptions == 0
