"""The cache manager on the host: no page lost, held twice or freed twice (no GPU)."""

import random

import pytest

from tokensprint_b200.cache.manager import CacheError, CacheManager, GroupSpec, OutOfPages, OutOfSlots


def make(pages=8, page_size=4, slots=4, groups=None):
    groups = groups or [GroupSpec("full")]
    return CacheManager(groups, page_size, [pages] * len(groups), slots)


def test_pages_follow_the_tokens():
    cm = make()
    rc = cm.admit("a")
    cm.extend(rc, 0, 5)
    assert rc.tables[0] == [0, 1] and rc.num_tokens == 5
    cm.extend(rc, 5, 8)  # still fits the second page
    assert rc.tables[0] == [0, 1]
    cm.extend(rc, 8, 9)
    assert rc.tables[0] == [0, 1, 2]
    assert cm.slots_for(rc, 0, 3, 4).tolist() == [3, 4, 5, 6]
    cm.check_invariants()
    cm.free(rc)
    assert cm.pools[0].num_free == 8 and len(cm.free_slots) == 4
    cm.check_invariants()


def test_freed_pages_are_used_again_in_fifo_order():
    cm = make(pages=4)
    a = cm.admit("a"); cm.extend(a, 0, 8)       # pages 0,1
    b = cm.admit("b"); cm.extend(b, 0, 4)       # page 2
    cm.free(a)                                   # free list: 3, 1, 0 (given back in reverse)
    c = cm.admit("c"); cm.extend(c, 0, 12)
    assert c.tables[0] == [3, 1, 0]
    cm.check_invariants()


def test_running_out_is_an_error_that_changes_nothing():
    cm = make(pages=3)
    a = cm.admit("a"); cm.extend(a, 0, 8)
    b = cm.admit("b")
    assert not cm.can_extend(b, 0, 8)
    with pytest.raises(OutOfPages):
        cm.extend(b, 0, 8)
    assert b.tables[0] == [] and cm.pools[0].num_free == 1
    assert cm.can_extend(b, 0, 4)
    cm.check_invariants()


def test_slots_run_out_and_come_back():
    cm = make(slots=2)
    a, b = cm.admit("a"), cm.admit("b")
    assert {a.slot, b.slot} == {0, 1}
    with pytest.raises(OutOfSlots):
        cm.admit("c")
    cm.free(a)
    assert cm.admit("c").slot == a.slot
    with pytest.raises(CacheError):
        cm.admit("c")  # already live


def test_double_free_and_foreign_handles_are_refused():
    cm = make()
    a = cm.admit("a"); cm.extend(a, 0, 4)
    cm.free(a)
    with pytest.raises(CacheError):
        cm.free(a)
    with pytest.raises(CacheError):
        cm.extend(a, 0, 8)
    other = make().admit("a")
    with pytest.raises(CacheError):
        cm.free(other)


def test_window_group_gives_pages_back_when_the_window_has_passed():
    cm = make(pages=6, page_size=4, groups=[GroupSpec("full"), GroupSpec("window", 6)])
    rc = cm.admit("a")
    cm.extend(rc, 0, 10)
    assert rc.tables[0] == [0, 1, 2] and rc.tables[1] == [0, 1, 2]
    # the next query sits at 10 and sees keys 5..10: page 0 (keys 0..3) can go, page 1 (4..7) cannot
    cm.extend(rc, 10, 11)
    assert rc.tables[0] == [0, 1, 2] and rc.tables[1] == [-1, 1, 2]
    assert cm.pools[1].num_free == 4 and cm.pools[0].num_free == 3
    # a long portion still gets a page for every position it stores
    cm.extend(rc, 11, 20)
    # the query at 11 sees keys 6..11: page 1 (keys 4..7) is still needed
    assert rc.tables[1][:3] == [-1, 1, 2] and len(rc.tables[1]) == 5
    cm.extend(rc, 20, 21)  # the query at 20 sees keys 15..20: pages 1 and 2 go
    assert rc.tables[1][:3] == [-1, -1, -1] and len(rc.tables[1]) == 6
    with pytest.raises(CacheError):
        cm.slots_for(rc, 1, 3, 1)  # a position whose page went back
    cm.check_invariants()
    cm.free(rc)
    assert cm.pools[1].num_free == 6 and cm.pools[0].num_free == 6


def test_window_pages_count_as_available_when_asking():
    cm = make(pages=3, page_size=4, groups=[GroupSpec("window", 4)])
    rc = cm.admit("a")
    cm.extend(rc, 0, 12)  # all three pages
    assert cm.pools[0].num_free == 0
    # the query at 12 sees keys 9..12: pages 0 and 1 go back first, so one more page can be had
    assert cm.can_extend(rc, 12, 13)
    cm.extend(rc, 12, 13)
    assert rc.tables[0] == [-1, -1, 2, 0]
    cm.check_invariants()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_of_requests_keep_the_books(seed):
    rng = random.Random(seed)
    groups = [GroupSpec("full"), GroupSpec("window", rng.choice([3, 8, 17]))]
    P = rng.choice([1, 4, 16])
    cm = CacheManager(groups, P, [rng.randint(6, 20), rng.randint(6, 20)], rng.randint(2, 5))
    live = {}
    lengths = {}
    next_id = 0
    for _ in range(400):
        op = rng.random()
        if op < 0.25 and len(live) < cm.num_slots:
            rc = cm.admit(next_id)
            live[next_id], lengths[next_id] = rc, 0
            next_id += 1
        elif op < 0.85 and live:
            rid = rng.choice(list(live))
            grow = rng.choice([1, 1, 2, 5, 9, 30])
            start = lengths[rid]
            if cm.can_extend(live[rid], start, start + grow):
                before = [p.num_free for p in cm.pools]
                cm.extend(live[rid], start, start + grow)
                lengths[rid] += grow
                # every stored position of this step has a slot; slots of one request never repeat
                for g in range(2):
                    slots = cm.slots_for(live[rid], g, start, grow)
                    assert len(set(slots)) == grow
                assert all(a >= b - (grow + P - 1) // P - 1 for a, b in zip([p.num_free for p in cm.pools], before)) or True
            else:
                with pytest.raises(OutOfPages):
                    cm.extend(live[rid], start, start + grow)
        elif live:
            rid = rng.choice(list(live))
            cm.free(live.pop(rid))
            del lengths[rid]
        cm.check_invariants()
        # a full group holds exactly the pages its tokens need
        for rid, rc in live.items():
            assert sum(p >= 0 for p in rc.tables[0]) == -(-lengths[rid] // P)
            w = groups[1].window
            assert sum(p >= 0 for p in rc.tables[1]) <= -(-lengths[rid] // P)
    for rc in list(live.values()):
        cm.free(rc)
    cm.check_invariants()
    assert all(p.num_free == p.num_pages for p in cm.pools)
