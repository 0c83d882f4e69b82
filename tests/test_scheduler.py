"""The scheduler's decisions, with a fake engine (the reference tests its scheduler the same way,
tests/test_scheduler.cpp:36-79): request N emits N, N+1, ...; pages are counted, nothing is computed."""
from typing import Dict

import pytest

from infer_b200.engine.scheduler import (BatchEngine, Request, SampleParams, Scheduler, SchedulerConfig, StopReason)


class FakeEngine(BatchEngine):
    def __init__(self, slots=2, max_seq=64, pages=1000, page=4):
        self.max_requests, self.max_seq_len, self.n_pages, self.page = slots, max_seq, pages, page
        self.len: Dict = {}
        self.batches = []

    def _pages(self, n):
        return -(-n // self.page)

    def _used(self, extra=()):
        lens = dict(self.len)
        for rid, n in extra:
            lens[rid] = lens.get(rid, 0) + n
        return sum(self._pages(n) for n in lens.values())

    def capacity_tokens(self): return self.n_pages * self.page
    def add_request(self, rid): assert rid not in self.len; self.len[rid] = 0
    def end_request(self, rid): del self.len[rid]
    def can_run(self, wanted): return self._used(wanted) <= self.n_pages
    def has_room(self, n): return self.n_pages - self._used() >= self._pages(n) + 1
    def tokens_that_fit(self, wanted, rid, n):
        while n > 0 and not self.can_run(list(wanted) + [(rid, n)]):
            n -= 1
        return n
    def pages_in_use(self): return self._used()
    def pages_total(self): return self.n_pages

    def run(self, batch):
        assert self.can_run([(b.rid, len(b.tokens)) for b in batch])
        self.batches.append([(b.rid, len(b.tokens), b.sample is not None) for b in batch])
        out = {}
        for b in batch:
            self.len[b.rid] += len(b.tokens)
            assert b.position == self.len[b.rid] - 1, "the sampler's key is the position of the last token fed"
            if b.sample is not None:
                out[b.rid] = 1000 * b.rid + self.len[b.rid]          # depends on request and position only
        return out


def _expected(rid, prompt_len, n):
    return [1000 * rid + prompt_len + i for i in range(n)]


def test_continuous_admits_as_slots_free_up():
    eng = FakeEngine(slots=2)
    sch = Scheduler(eng, SchedulerConfig())
    for rid, mn in ((1, 2), (2, 7), (3, 3)):
        sch.submit(Request(rid, [7] * 3, mn))
    sch.run_until_idle()
    done = {c.id: c for c in sch.completed}
    assert [c.id for c in sch.completed] == [1, 3, 2]
    assert all(done[r].reason == StopReason.MAX_NEW for r in done)
    assert done[2].tokens == _expected(2, 3, 7) and done[3].tokens == _expected(3, 3, 3)
    assert done[3].admitted_step == done[1].finished_step + 1       # the freed slot is refilled at once
    assert eng.len == {} and eng.pages_in_use() == 0


def test_static_waits_for_the_whole_batch():
    eng = FakeEngine(slots=2)
    sch = Scheduler(eng, SchedulerConfig(continuous=False))
    for rid, mn in ((1, 2), (2, 6), (3, 2)):
        sch.submit(Request(rid, [7] * 3, mn))
    sch.run_until_idle()
    done = {c.id: c for c in sch.completed}
    assert done[3].admitted_step > done[2].finished_step


def test_prompts_are_cut_under_the_token_budget_and_decodes_go_first():
    eng = FakeEngine(slots=3, max_seq=200)
    sch = Scheduler(eng, SchedulerConfig(max_batch_tokens=8))
    sch.submit(Request(1, [1] * 3, 4))
    sch.step()                                               # request 1 prefilled (3 tokens), first token sampled
    sch.submit(Request(2, [2] * 20, 2))
    sch.step()
    assert eng.batches[-1] == [(1, 1, True), (2, 7, False)]  # one decode token first, then 7 of the budget of 8
    sch.step()
    assert eng.batches[-1] == [(1, 1, True), (2, 7, False)]
    sch.step()
    assert eng.batches[-1][-1] == (2, 6, True)               # the last portion ends the prompt: it samples
    sch.run_until_idle()
    done = {c.id: c.tokens for c in sch.completed}
    assert done[1] == _expected(1, 3, 4) and done[2] == _expected(2, 20, 2)
    assert all(sum(n for _, n, _ in b) <= 8 for b in eng.batches)


def test_eos_max_new_arrival_and_cancel():
    eng = FakeEngine(slots=2)
    tokens = []
    sch = Scheduler(eng, SchedulerConfig(eos_id=1005, on_token=lambda r, t: tokens.append((r, t))))
    sch.submit(Request(1, [0] * 3, 10))                      # emits 1003, 1004, 1005 = eos
    sch.submit(Request(3, [0] * 2, 50))
    sch.submit(Request(2, [0] * 2, 3, arrival_step=4))      # FIFO: what is queued behind it waits too
    sch.submit(Request(4, [0] * 2, 5, eos_id=-1))
    sch.cancel(4)                                            # cancelled while queued: never runs
    for _ in range(3):
        sch.step()
    sch.cancel(3)                                            # cancelled while active
    sch.run_until_idle()
    done = {c.id: c for c in sch.completed}
    assert done[1].reason == StopReason.EOS and done[1].tokens == [1003, 1004, 1005]
    assert done[2].reason == StopReason.MAX_NEW and done[2].admitted_step >= 4
    assert done[3].reason == StopReason.CANCELLED and 0 < len(done[3].tokens) < 50
    assert done[4].reason == StopReason.CANCELLED and done[4].tokens == []
    assert (1, 1005) in tokens and eng.len == {}


def test_request_that_cannot_fit_is_refused_at_submit():
    eng = FakeEngine(slots=2, max_seq=16)
    sch = Scheduler(eng)
    with pytest.raises(ValueError, match="does not fit"):
        sch.submit(Request(1, [0] * 10, 7))
    with pytest.raises(ValueError, match="does not fit"):
        Scheduler(FakeEngine(max_seq=100, pages=3, page=4)).submit(Request(1, [0] * 10, 7))
    with pytest.raises(ValueError, match="empty"):
        sch.submit(Request(2, [], 3))


def test_pages_run_out_youngest_is_preempted_and_outputs_are_unchanged():
    # 3 requests of 8 + 12 tokens need 5 pages each at the end; the pool has 9.
    eng = FakeEngine(slots=3, max_seq=64, pages=9, page=4)
    sch = Scheduler(eng, SchedulerConfig(max_batch_tokens=64))
    for rid in (1, 2, 3):
        sch.submit(Request(rid, [0] * 8, 12))
    sch.run_until_idle()
    done = {c.id: c for c in sch.completed}
    assert sch.preemptions > 0
    assert max(c.preemptions for c in sch.completed) > 0 and done[1].preemptions == 0   # the oldest is never the victim
    for rid in (1, 2, 3):
        assert done[rid].tokens == _expected(rid, 8, 12), "a preempted request resumes with the same stream"
    assert eng.len == {} and eng.pages_in_use() == 0
    kinds = [sch.events[i].kind for i in range(len(sch.events))]
    assert "preempt" in kinds and kinds.count("retire") == 3


def test_prompt_portion_is_shortened_to_the_free_pages():
    eng = FakeEngine(slots=2, max_seq=64, pages=6, page=4)
    sch = Scheduler(eng, SchedulerConfig(max_batch_tokens=64))
    sch.submit(Request(1, [0] * 12, 4))
    sch.step()                                               # 3 pages taken
    eng.n_pages = 5                                          # the pool shrinks under the scheduler: 2 pages free
    sch.active[1]                                            # still active
    sch.submit(Request(2, [0] * 10, 2))
    # request 2 is not admitted while there is no room for its prompt and one more page
    sch.step()
    assert 2 not in sch.active
    eng.n_pages = 8
    sch.step()
    assert 2 in sch.active
    sch.run_until_idle()
    assert {c.id: c.tokens for c in sch.completed}[2] == _expected(2, 10, 2)


def test_event_ring_wraps():
    eng = FakeEngine(slots=1)
    sch = Scheduler(eng, SchedulerConfig(event_capacity=4))
    sch.submit(Request(1, [0] * 2, 10))
    sch.run_until_idle()
    assert len(sch.events) == 4 and sch.events.dropped > 0
    assert sch.events[3].kind == "step" and sch.events[2].kind == "retire"


@pytest.mark.parametrize("pages", [1000, 9])
def test_overlap_mode_gives_the_same_streams(pages):
    """Launching a step before the previous step's tokens are read changes when tokens are seen, not what they are;
    with few pages the tokens in flight are read before a victim is chosen."""
    def run(overlap):
        eng = FakeEngine(slots=3, max_seq=64, pages=pages, page=4)
        seen = []
        sch = Scheduler(eng, SchedulerConfig(max_batch_tokens=16, overlap=overlap, eos_id=2012 if pages == 1000 else -1,
                                             on_token=lambda r, t: seen.append((r, t))))
        for rid, plen, mn in ((1, 8, 12), (2, 8, 12), (3, 5, 9), (4, 20, 3)):
            sch.submit(Request(rid, [0] * plen, mn))
        sch.run_until_idle()
        assert eng.len == {} and eng.pages_in_use() == 0 and sch.idle()
        return {c.id: (c.reason, c.tokens) for c in sch.completed}, seen, sch
    plain, seen_p, _ = run(False)
    over, seen_o, sch = run(True)
    assert plain == over
    if pages == 1000:
        assert plain[2] == (StopReason.EOS, [2008, 2009, 2010, 2011, 2012])      # eos is honoured although it is seen late
    assert sorted(seen_p) == sorted(seen_o)
    for rid in (1, 2, 3, 4):
        assert [t for r, t in seen_o if r == rid] == over[rid][1]          # per request, tokens are reported in order
    if pages == 9:
        assert sch.preemptions > 0


def test_overlap_decode_items_carry_the_feedback_token():
    from infer_b200.engine.scheduler import FEEDBACK_TOKEN
    eng = FakeEngine(slots=1)
    fed = []
    orig = eng.run
    eng.run = lambda batch: (fed.append([b.tokens for b in batch]), orig(batch))[1]
    sch = Scheduler(eng, SchedulerConfig(overlap=True))
    sch.submit(Request(1, [5, 6, 7], 4))
    sch.run_until_idle()
    assert fed[0] == [[5, 6, 7]] and all(step == [[FEEDBACK_TOKEN]] for step in fed[1:4])
    assert sch.completed[0].tokens == _expected(1, 3, 4)
