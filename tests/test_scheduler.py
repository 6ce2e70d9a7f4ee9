"""The scheduler's decisions with no model behind it (no GPU)."""
import random

import pytest

from rust_mlx_b200.cache import GroupGeometry, PageTable
from rust_mlx_b200.engine.scheduler import RequestRejected, Scheduler


def make(pages=64, page=4, max_seqs=4, budget=16, chunk=8, max_context=0, window=0):
    table = PageTable([GroupGeometry(pages, page, window)], max_requests=max_seqs)
    return table, Scheduler(table, max_seqs=max_seqs, max_batch_tokens=budget, prefill_chunk=chunk, max_context=max_context)


def run(table, s, lengths, finish_after, record=None):
    """Drive to completion; every request generates finish_after[r] tokens."""
    made = {r: 0 for r in lengths}
    steps = 0
    while not s.idle():
        entries = s.next()
        assert entries, "an idle-less scheduler must make progress"
        if record is not None:
            record.append(entries)
        assert len({e.req for e in entries}) == len(entries)
        for e in entries:
            assert table.reserved(e.req) >= e.start + e.count
        s.step_done()
        for e in entries:
            assert table.length(e.req) == e.start + e.count
            if e.wants_logits:
                made[e.req] += 1
                if made[e.req] >= finish_after[e.req]:
                    s.finish(e.req)
                else:
                    s.append_token(e.req)
        table.check()
        steps += 1
        assert steps < 10000
    return made


def test_prompts_are_cut_under_the_budget_and_decodes_come_first():
    table, s = make(budget=10, chunk=6)
    s.add(0, 3, 4)
    s.add(1, 20, 2)
    log = []
    made = run(table, s, {0: 3, 1: 20}, {0: 4, 1: 2}, log)
    assert made == {0: 4, 1: 2}
    first = log[0]
    assert [(e.req, e.start, e.count, e.wants_logits) for e in first] == [(0, 0, 3, True), (1, 0, 6, False)]
    second = log[1]
    # request 0 decodes one token (listed first), request 1 goes on with its prompt
    assert (second[0].req, second[0].count, second[0].wants_logits) == (0, 1, True)
    assert (second[1].req, second[1].start, second[1].count) == (1, 6, 6)
    for entries in log:
        assert sum(e.count for e in entries) <= 10
        assert all(e.count <= 6 for e in entries)
    assert table.free_pages(0) == 64 and table.live() == 0


def test_admission_waits_for_a_free_seat():
    table, s = make(max_seqs=2, budget=64, chunk=64)
    for r in range(4):
        s.add(r, 5, 3)
    entries = s.next()
    assert [e.req for e in entries] == [0, 1] and s.waiting == 2
    s.step_done()
    s.finish(0)
    s.append_token(1)
    entries = s.next()
    assert [e.req for e in entries] == [1, 2]
    s.step_done()


def test_rejections():
    table, s = make(pages=4, page=4, max_context=32)
    with pytest.raises(RequestRejected, match="empty"):
        s.add(0, 0, 5)
    with pytest.raises(RequestRejected, match="context"):
        s.add(0, 30, 5)
    with pytest.raises(RequestRejected, match="pages"):
        s.add(0, 10, 8)           # 17 tokens in the cache need 5 pages of 4
    s.add(0, 10, 7)               # 16 tokens fit exactly
    with pytest.raises(RequestRejected, match="in use"):
        s.add(0, 3, 1)


def test_when_pages_run_out_the_request_admitted_last_steps_back_and_is_computed_again():
    table, s = make(pages=6, page=4, max_seqs=3, budget=32, chunk=32)
    s.add(0, 8, 12)               # will need 5 pages in the end
    s.add(1, 8, 12)
    log = []
    made = run(table, s, {0: 8, 1: 8}, {0: 12, 1: 12}, log)
    assert made[0] == 12          # request 0 is never disturbed
    # request 1 was preempted at least once: it shows up again from position 0 with more tokens than its prompt
    restarts = [e for entries in log for e in entries if e.req == 1 and e.start == 0]
    assert len(restarts) >= 2 and restarts[-1].count > 8
    assert table.free_pages(0) == 6
    # request 0's entries are contiguous: every start is the previous end
    at = 0
    for entries in log:
        for e in entries:
            if e.req == 0:
                assert e.start == at
                at += e.count


def test_preemption_is_reported():
    table, s = make(pages=4, page=4, max_seqs=2, budget=32, chunk=32)
    s.add(0, 7, 8)
    s.add(1, 7, 8)
    seen = []
    made = {0: 0, 1: 0}
    while not s.idle():
        entries = s.next()
        seen += s.take_preempted()
        s.step_done()
        for e in entries:
            if e.wants_logits:
                made[e.req] += 1
                (s.finish if made[e.req] >= 8 else s.append_token)(e.req)
    assert seen and set(seen) == {1}


def test_a_window_group_lets_long_requests_share_few_pages():
    table, s = make(pages=8, page=4, max_seqs=2, budget=8, chunk=4, window=6)
    s.add(0, 40, 10)
    s.add(1, 33, 10)
    made = run(table, s, {0: 40, 1: 33}, {0: 10, 1: 10})
    assert made == {0: 10, 1: 10}


@pytest.mark.parametrize("seed", range(6))
def test_random_workloads_finish_with_every_page_back(seed):
    rng = random.Random(seed)
    pages, page = rng.randrange(12, 40), rng.choice([2, 4, 8])
    table, s = make(pages=pages, page=page, max_seqs=rng.randrange(1, 5), budget=rng.randrange(4, 40),
                    chunk=rng.randrange(1, 20))
    lengths, gen = {}, {}
    r = 0
    while len(lengths) < 12:
        p, g = rng.randrange(1, 50), rng.randrange(1, 20)
        try:
            s.add(r, p, g)
            lengths[r], gen[r] = p, g
        except RequestRejected:
            assert -(-(p + g - 1) // page) > pages
        r += 1
    made = run(table, s, lengths, gen)
    assert made == gen
    assert table.free_pages(0) == pages and table.live() == 0


def test_requests_that_await_their_token_are_not_disturbed():
    """A step may be asked for while the last step's tokens are not read yet (the caller runs ahead): requests
    whose next token is not known have nothing to feed; that is no reason to take their pages away."""
    table, s = make(pages=8, page=4, max_seqs=3, budget=32, chunk=32)
    s.add(0, 5, 4)
    s.add(1, 6, 4)
    assert [e.req for e in s.next()] == [0, 1]
    s.step_done()
    assert s.next() == [] and s.take_preempted() == []          # both await their first token
    s.append_token(0)                                            # request 0's token is on its way: it may run ahead
    entries = s.next()
    assert [(e.req, e.start, e.count) for e in entries] == [(0, 5, 1)] and s.take_preempted() == []
    s.step_done()
    s.finish(1)                                                  # request 1's token turned out to end it
    s.append_token(0)
    assert [(e.req, e.start) for e in s.next()] == [(0, 6)]
    s.step_done()
    s.finish(0)
    assert s.idle() and table.free_pages(0) == 8
