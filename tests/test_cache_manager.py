"""The cache manager (no GPU): no page lost, held twice or freed twice, under random orders of
requests; the null page is never handed out; freed pages are used again in the order of their
release; window groups give pages back as the window passes them."""

from __future__ import annotations

import random

import numpy as np
import pytest

from research_2_b200.cache import CacheError, CacheManager, GroupSpec, OutOfPages
from research_2_b200.engine.batch import BatchLimits, batch_for


def test_pages_come_in_order_and_never_the_null_page():
    cm = CacheManager([GroupSpec(4, 0, 6)], 3, 24)
    cm.open(0)
    cm.reserve(0, 0, 9)
    assert list(cm.table(0)) == [1, 2, 3, 0, 0, 0]
    assert cm.n_free() == 3 and cm.pages_held(0) == 3
    cm.reserve(0, 9, 12)  # still inside page 3
    assert cm.pages_held(0) == 3
    cm.reserve(0, 12, 13)
    assert list(cm.table(0))[:4] == [1, 2, 3, 4]
    assert cm.check() == ""


def test_freed_pages_are_reused_in_the_order_of_their_release():
    cm = CacheManager([GroupSpec(2, 0, 6)], 3, 12)
    cm.open(0); cm.open(1)
    cm.reserve(0, 0, 4)   # pages 1 2
    cm.reserve(1, 0, 4)   # pages 3 4
    cm.close(0)           # free list: 5 6 1 2
    cm.open(2)
    cm.reserve(2, 0, 8)
    assert list(cm.table(2))[:4] == [5, 6, 1, 2]
    assert cm.check() == "" and cm.n_free() == 0


def test_all_or_nothing_when_pages_run_out():
    cm = CacheManager([GroupSpec(4, 0, 3), GroupSpec(4, 0, 2)], 2, 16)
    cm.open(0)
    assert not cm.can_reserve(0, 0, 12)  # the second group has only two pages
    with pytest.raises(OutOfPages):
        cm.reserve(0, 0, 12)
    assert cm.n_free(0) == 3 and cm.n_free(1) == 2 and cm.pages_held(0, 0) == 0
    cm.reserve(0, 0, 8)
    assert cm.can_reserve(0, 8, 8, spare_pages=0) and not cm.can_reserve(0, 8, 8, spare_pages=1)


def test_errors_are_reported_not_fatal():
    cm = CacheManager([GroupSpec(4, 0, 3)], 2, 8)
    with pytest.raises(CacheError):
        cm.close(0)  # never opened
    cm.open(0)
    with pytest.raises(CacheError):
        cm.open(0)  # opened twice
    with pytest.raises(CacheError):
        cm.reserve(0, 0, 9)  # beyond max_seq_len
    with pytest.raises(CacheError):
        cm.open(5)
    cm.close(0)
    with pytest.raises(CacheError):
        cm.close(0)  # a second close frees nothing twice
    assert cm.n_free() == 3 and cm.check() == ""
    with pytest.raises(ValueError):
        CacheManager([GroupSpec(0, 0, 3)], 2, 8)


def test_window_group_gives_pages_back_as_the_window_passes():
    cm = CacheManager([GroupSpec(4, 0, 16), GroupSpec(4, 6, 5)], 1, 64)
    cm.open(0)
    held = []
    for start in range(0, 40, 3):
        cm.slide(0, start)
        cm.reserve(0, start, start + 3)
        table = cm.table(0, 1)
        first_key = max(0, start - 6 + 1)
        assert all(table[i] == 0 for i in range(first_key // 4)), "a page behind the window is still held"
        assert all(table[i] != 0 for i in range(first_key // 4, -(-(start + 3) // 4))), "a page in the window is missing"
        held.append(cm.pages_held(0, 1))
        assert cm.pages_held(0, 0) == -(-(start + 3) // 4)
        assert cm.check() == ""
    assert max(held) <= cm.worst_pages(1, 64, 3) <= 5
    cm.close(0)
    assert cm.n_free(0) == 16 and cm.n_free(1) == 5


def test_fill_batch_slots_tables_and_state():
    cm = CacheManager([GroupSpec(4, 0, 8), GroupSpec(2, 0, 16)], 3, 16)
    cm.open(2); cm.open(0)
    cm.reserve(2, 0, 7)
    cm.reserve(0, 0, 3)
    b = batch_for(cm.table_widths, 6, 2, 2)
    b.set_entries([2, 0], [4, 0], [[9, 9, 9], [5, 6, 7]])
    cm.fill(b)
    b.pad()
    assert list(b.positions[:6]) == [4, 5, 6, 0, 1, 2]
    assert list(b.row_entry[:6]) == [0, 0, 0, 1, 1, 1]
    assert list(b.q_start[:3]) == [0, 3, 6] and list(b.seq_lens[:2]) == [7, 3]
    assert list(b.fresh[:2]) == [0, 1] and list(b.state_slot[:2]) == [2, 0]
    t2, t0 = cm.table(2, 0), cm.table(0, 0)
    assert list(b.slot_mapping[0, :6]) == [t2[1] * 4 + 0, t2[1] * 4 + 1, t2[1] * 4 + 2, t0[0] * 4, t0[0] * 4 + 1, t0[0] * 4 + 2]
    u2 = cm.table(2, 1)
    assert list(b.slot_mapping[1, :3]) == [u2[2] * 2, u2[2] * 2 + 1, u2[3] * 2]
    assert np.array_equal(b.block_tables[0][0], t2) and np.array_equal(b.block_tables[1][1], cm.table(0, 1))
    b.check(BatchLimits(100, 16, [GroupSpec(4, 0, 8), GroupSpec(2, 0, 16)], cm.table_widths))
    b2 = batch_for(cm.table_widths, 4, 1, 1)
    b2.set_entries([0], [3], [[1, 2, 3, 4]])  # positions 3..6 were never reserved
    with pytest.raises(OutOfPages):
        cm.fill(b2)


def test_a_batch_that_the_caller_filled_is_checked_against_the_pool():
    """Each refusal of the host-side check, on a batch that is sound but for one value; the second
    group's arrays lie behind the first's in the buffer."""
    groups = [GroupSpec(4, 0, 8), GroupSpec(2, 0, 16)]
    cm = CacheManager(groups, 3, 16)
    cm.open(2); cm.open(0)
    cm.reserve(2, 0, 7)
    cm.reserve(0, 0, 3)
    b = batch_for(cm.table_widths, 8, 3, 3)  # capacities beyond the counts
    b.set_entries([2, 0], [4, 0], [[9, 9, 9], [5, 6, 7]])
    cm.fill(b)
    b.pad()
    limits = BatchLimits(10, 16, groups, cm.table_widths)
    b.check(limits)

    def refused(array, index, value, error, text):
        before = array[index]
        array[index] = value
        with pytest.raises(error, match=text):
            b.check(limits)
        array[index] = before
        b.check(limits)

    refused(b.row_entry, 4, 2, AssertionError, "a row names an entry outside the batch")
    refused(b.row_entry, 4, -1, AssertionError, "a row names an entry outside the batch")
    refused(b.row_entry, 3, 0, AssertionError, "entry 0: rows are not its newest positions")
    refused(b.positions, 5, 3, AssertionError, "entry 1: rows are not its newest positions")
    refused(b.seq_lens, 0, 8, AssertionError, "entry 0: rows are not its newest positions")
    refused(b.input_ids, 2, 10, ValueError, "outside the vocabulary")
    refused(b.input_ids, 2, -1, ValueError, "outside the vocabulary")
    refused(b.slot_mapping[0], 1, 3, ValueError, "group 0: a slot lies outside the pool or in the null page")
    refused(b.slot_mapping[0], 1, 9 * 4, ValueError, "group 0: a slot lies outside the pool")
    refused(b.slot_mapping[1], 5, 17 * 2, ValueError, "group 1: a slot lies outside the pool")
    refused(b.block_tables[0], (1, 3), 9, ValueError, "group 0: a block table names a page outside the pool")
    refused(b.block_tables[1], (0, 7), -1, ValueError, "group 1: a block table names a page outside the pool")
    with pytest.raises(ValueError, match="beyond max_seq_len"):
        b.check(BatchLimits(10, 6, groups, cm.table_widths))
    # (what lies beyond the counts is padding and is not looked at)
    b.block_tables[1][2, 0] = 99
    b.slot_mapping[1, 7] = 999
    b.check(limits)


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_every_invariant(seed):
    rng = random.Random(seed)
    groups = [GroupSpec(rng.choice([2, 4, 8]), 0, rng.randint(6, 20)), GroupSpec(4, rng.choice([0, 5, 9]), rng.randint(4, 12))]
    n_req, max_len = 5, 48
    cm = CacheManager(groups, n_req, max_len)
    fed = {}
    for _ in range(600):
        r = rng.randrange(n_req)
        action = rng.random()
        if r not in fed:
            cm.open(r)
            fed[r] = 0
        elif action < 0.15:
            cm.close(r)
            del fed[r]
        else:
            n = rng.randint(1, 7)
            total = min(max_len, fed[r] + n)
            cm.slide(r, fed[r])
            if cm.can_reserve(r, fed[r], total):
                before = [cm.n_free(g) for g in range(2)]
                cm.reserve(r, fed[r], total)
                assert all(cm.n_free(g) <= before[g] for g in range(2))
                fed[r] = total
            else:
                before = [cm.n_free(g) for g in range(2)]
                with pytest.raises(OutOfPages):
                    cm.reserve(r, fed[r], total)
                assert [cm.n_free(g) for g in range(2)] == before, "a refused reservation took pages"
        assert cm.check() == "", cm.check()
        seen = [set(), set()]
        for q in fed:  # no page in two live tables, and never the null page among the held ones
            for g in range(2):
                pages = [p for p in cm.table(q, g) if p != 0]
                assert len(pages) == cm.pages_held(q, g)
                assert not (seen[g] & set(pages))
                seen[g] |= set(pages)
        for g in range(2):
            assert len(seen[g]) + cm.n_free(g) == groups[g].num_pages
    for r in list(fed):
        cm.close(r)
    assert [cm.n_free(g) for g in range(2)] == [groups[0].num_pages, groups[1].num_pages]


def test_the_replay_tests_mixed_traces_use_pages_again():
    """The GPU tests replay their mixed traces in a pool of the trace's own peak demand plus one page.
    Over the cache manager alone (no GPU) that pool is enough, and at least a third of its pages
    pass from one request to another, at every configuration that those tests use."""
    from tests import traces
    from tests.helpers import TINY, random_tokens
    from tests.test_odd_shapes_gpu import ODD
    from tests.test_replay_gpu import LENGTHS

    cases = [(name, TINY[name]["page_size"], 4, [(100 + i, n) for i, n in enumerate(LENGTHS[name])]) for name in LENGTHS]
    cases += [(name, t["page_size"], 2, [(300 + i, n) for i, n in enumerate(t["lengths"])]) for name, t in ODD.items()]
    cases.append(("124M", 16, 3, [(500 + i, n) for i, n in enumerate((130, 40, 9, 200, 70, 25))]))
    for name, page, live, lengths in cases:
        requests = {f"r{i}": random_tokens(seed, n, 50) for i, (seed, n) in enumerate(lengths)}
        tb = traces.mixed(requests, max_live=live)
        pool = traces.peak_pages(tb, page) + 1
        owners = traces.page_traffic(tb, page, pool)   # raises OutOfPages if the pool were too small
        reused = sum(len(seen) >= 2 for seen in owners.values())
        assert 3 * reused >= pool, f"{name}: {reused} of {pool} pages are used again"
