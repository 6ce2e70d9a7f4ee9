"""The cache manager's bookkeeping (no GPU): no page lost, held twice or freed twice."""
import random

import pytest

from rust_mlx_b200.cache import CacheError, GroupGeometry, OutOfPages, OutOfSlots, PageTable


def held_pages(t, reqs, g=0):
    return [p for r in reqs for p in t.table(r, g) if p >= 0]


def test_pages_follow_length_and_come_back():
    t = PageTable([GroupGeometry(6, 8)], max_requests=3)
    assert t.open(1) == 0 and t.open(2) == 1
    t.reserve(1, 9)                       # two pages
    assert t.table(1, 0) == [0, 1] and t.free_pages(0) == 4
    t.commit(1, 9)
    t.reserve(1, 16)                      # still two pages
    assert t.table(1, 0) == [0, 1]
    t.reserve(2, 1)
    assert t.table(2, 0) == [2]
    t.commit(1, 16)
    t.reserve(1, 17)
    assert t.table(1, 0) == [0, 1, 3]
    assert t.close(1) == 3 and t.free_pages(0) == 5
    t.open(3)
    t.reserve(3, 8)
    assert t.table(3, 0) == [3]           # the page freed last is used again first
    t.check()


def test_reserve_is_all_or_nothing_over_groups():
    t = PageTable([GroupGeometry(4, 8), GroupGeometry(2, 8)], max_requests=2)
    t.open(1)
    with pytest.raises(OutOfPages):
        t.reserve(1, 17)                  # 3 pages: the second group has 2
    assert t.free_pages(0) == 4 and t.free_pages(1) == 2 and t.reserved(1) == 0
    assert t.max_reservable(1, 100) == 16
    t.reserve(1, 16)
    assert t.try_reserve(1, 17) is False
    t.check()


def test_errors():
    t = PageTable([GroupGeometry(2, 4)], max_requests=1)
    t.open(5)
    with pytest.raises(CacheError):
        t.open(5)
    with pytest.raises(OutOfSlots):
        t.open(6)
    with pytest.raises(CacheError):
        t.reserve(7, 1)
    t.reserve(5, 4)
    with pytest.raises(CacheError):
        t.commit(5, 5)                    # beyond what was reserved
    t.commit(5, 4)
    with pytest.raises(CacheError):
        t.reserve(5, 3)                   # shrinking
    t.close(5)
    with pytest.raises(CacheError):
        t.close(5)                        # freed twice
    with pytest.raises(CacheError):
        PageTable([GroupGeometry(2, 0)], max_requests=1)
    t.check()


def test_release_reserved_gives_back_what_a_failed_step_took():
    t = PageTable([GroupGeometry(8, 4)], max_requests=2)
    t.open(1)
    t.reserve(1, 6)
    t.commit(1, 6)
    t.reserve(1, 20)
    assert t.free_pages(0) == 3
    assert t.release_reserved(1) == 3
    assert t.free_pages(0) == 6 and t.reserved(1) == 6 and t.table(1, 0) == [0, 1]
    t.check()


def test_a_window_gives_pages_back_as_it_passes_them():
    # group 0 keeps everything, group 1 reads the last 10 positions only
    t = PageTable([GroupGeometry(16, 4), GroupGeometry(16, 4, window=10)], max_requests=1)
    t.open(1)
    n = 0
    for step in (7, 2, 13, 1, 1, 1, 9):
        t.reserve(1, n + step)
        # during the step the group still holds every page from the window before the portion on
        first_needed = max(0, n - 10 + 1)
        tab = t.table(1, 1)
        assert all(tab[i] >= 0 for i in range(first_needed // 4, len(tab)))
        n += step
        t.commit(1, n)
        tab = t.table(1, 1)
        dead = max(0, n - 10 + 1) // 4
        assert all(p == -1 for p in tab[:dead]) and all(p >= 0 for p in tab[dead:])
        assert len(t.table(1, 0)) == -(-n // 4) and all(p >= 0 for p in t.table(1, 0))
        t.check()
    assert t.pages_held(1, 1) <= 4
    t.close(1)
    assert t.free_pages(1) == 16
    t.check()


def test_peak_pages():
    t = PageTable([GroupGeometry(100, 8), GroupGeometry(100, 8, window=16)], max_requests=1)
    assert t.peak_pages(0, 100, 32) == 13
    assert t.peak_pages(1, 10, 32) == 2
    assert t.peak_pages(1, 1000, 1) <= 4
    assert t.peak_pages(1, 1000, 32) <= 8


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_of_requests_keep_the_books_right(seed):
    rng = random.Random(seed)
    groups = [GroupGeometry(rng.randrange(6, 40), rng.choice([4, 8, 16])),
              GroupGeometry(rng.randrange(6, 40), rng.choice([4, 8, 16]), window=rng.randrange(3, 40))]
    t = PageTable(groups, max_requests=5)
    live = {}
    next_id = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            t.open(next_id)
            live[next_id] = 0
            next_id += 1
        elif op < 0.85 and live:
            r = rng.choice(list(live))
            grow = rng.randrange(1, 30)
            if t.try_reserve(r, live[r] + grow):
                if rng.random() < 0.1:
                    t.release_reserved(r)           # the step did not run after all
                else:
                    live[r] += grow
                    t.commit(r, live[r])
            else:
                assert t.reserved(r) == max(live[r], t.reserved(r))
        elif live:
            r = rng.choice(list(live))
            t.close(r)
            del live[r]
        t.check()
        for g in range(2):
            held = held_pages(t, live, g)
            assert len(held) == len(set(held))
            assert len(held) + t.free_pages(g) == groups[g].num_pages
        for r, n in live.items():
            assert t.length(r) == n
        assert t.live() == len(live) and t.free_slots() == 5 - len(live)
        assert len({t.slot(r) for r in live}) == len(live)
    for r in list(live):
        t.close(r)
    assert all(t.free_pages(g) == groups[g].num_pages for g in range(2))
