"""
The cache manager on the host, against a storage fake whose slots hold token ids (no GPU): prefix
reuse, partial copies, copy on write, dedupe, eviction order, window release, state slots, forks,
and random workloads with the whole contract checked after every operation.
"""

import random

import pytest

from cache_fakes import FakeStorage, check_invariants, layout_of
from tinyserve_llm_b200.cache import CacheFull, CacheManager, PagePool, PrefixIndex, plan_layout, shared_run
from tinyserve_llm_b200.parts.base import KVNeed


def make(pages=8, page_tokens=4, windows=(0,), caching=True, state_bytes=0, slots=0):
    layout = layout_of(page_tokens, windows, state_bytes)
    counts = [pages] * len(windows)
    storage = FakeStorage(layout, counts, slots)
    return CacheManager(layout, counts, storage, caching=caching, num_state_slots=slots), storage


def run(manager, storage, seq_id, tokens, chunk=None):
    """Admit and feed all tokens (in portions of `chunk`), committing each step."""
    assert manager.admit(seq_id, tokens, chunk)
    while True:
        storage.run_step(manager, seq_id)
        seq = manager.seqs[seq_id]
        manager.commit(seq_id, seq.reserved - seq.committed)
        check_invariants(manager, storage)
        done = manager.committed_tokens(seq_id)
        if done == len(tokens):
            return
        manager.extend(seq_id, tokens[done:done + (chunk or len(tokens))])


def decode(manager, storage, seq_id, token):
    manager.extend(seq_id, [token])
    storage.run_step(manager, seq_id)
    manager.commit(seq_id, 1)
    check_invariants(manager, storage)


# ----------------------------------------------------------------------------- the index and the pool
def test_shared_run_counts_leading_tokens():
    assert shared_run((1, 2, 3), (1, 2, 3)) == 3 and shared_run((1, 2, 3), (1, 2, 9, 9)) == 2
    assert shared_run((), (1,)) == 0 and shared_run((5,), (6,)) == 0 and shared_run((1, 2, 3, 4, 5, 6, 7), (1, 2, 3, 4, 5, 9, 7)) == 5


def test_the_nearest_pages_are_neighbours_in_the_sorted_list():
    index = PrefixIndex(4)
    a = index.file(index.root, 0, (1, 2, 3))
    b = index.file(index.root, 1, (1, 2, 9, 9))
    c = index.file(index.root, 2, (1, 5))
    d = index.file(index.root, 3, (0, 7))
    assert [e.tokens for e in index.root.after] == [(0, 7), (1, 2, 3), (1, 2, 9, 9), (1, 5)]
    assert index.nearest(index.root, (1, 2, 3, 4)) == (3, [a])
    run, pages = index.nearest(index.root, (1, 2))
    assert run == 2 and set(pages) == {a, b}
    assert index.nearest(index.root, (7,)) == (0, []) and index.nearest(index.root, (1, 6)) [0] == 1
    assert set(index.nearest(index.root, (1, 6))[1]) == {a, b, c}
    index.drop(a)
    assert index.nearest(index.root, (1, 2, 3)) == (2, [b]) and len(index) == 3 and d.before is index.root


def test_lookup_never_takes_the_last_token_and_honours_a_limit():
    index = PrefixIndex(4)
    first = index.file(index.root, 0, (1, 2, 3, 4))
    index.file(first, 1, (5, 6))
    assert index.lookup([1, 2, 3, 4]).num_tokens == 3              # the last token is left to run (a run of 3 to copy)
    assert index.lookup([1, 2, 3, 4, 5]).num_tokens == 4
    whole = index.lookup([1, 2, 3, 4, 5, 6, 7])
    assert whole.num_tokens == 6 and [p.page for p in whole.pages] == [0, 1] and whole.run == 0
    assert index.lookup([1, 2, 3, 4, 5, 6, 7], limit=5).num_tokens == 5
    assert index.lookup([1, 2, 3, 4, 5, 6, 7], limit=0).num_tokens == 0
    partial = index.lookup([1, 2, 9, 9, 9])
    assert partial.run == 2 and partial.pages == [] and [p.page for p in partial.starting_with_run] == [0]


def test_a_page_that_gains_tokens_moves_in_the_order_and_meets_its_twin():
    index = PrefixIndex(4)
    a = index.file(index.root, 0, (1, 2))
    b = index.file(index.root, 1, (1, 2, 0, 5))
    assert index.file(index.root, 7, (1, 2)) is a                 # the same tokens again: the page on record is kept
    assert index.lengthen(a, (1, 2, 3)) is a and [e.page for e in index.root.after] == [1, 0]
    assert index.lengthen(a, (1, 2, 3, 4)) is a
    c = index.file(index.root, 2, (1, 2, 0))
    assert index.lengthen(c, (1, 2, 0, 5)) is b and c.tokens == (1, 2, 0)


def test_the_pool_evicts_the_stalest_end_of_a_chain_and_wakes_idle_pages():
    index = PrefixIndex(2)
    pool = PagePool(4, index)
    pages = [pool.take() for _ in range(3)]
    assert pages == [0, 1, 2] and pool.available() == 1
    first = index.file(index.root, 0, (1, 2))
    second = index.file(first, 1, (3, 4))
    for page in (2, 1, 0):                                         # from the end, as a released request does
        pool.let_go(page)
    assert pool.blank_pages() == [3, 2] and sorted(pool.idle_pages()) == [0, 1] and pool.available() == 4
    assert [pool.take(), pool.take()] == [2, 3]
    assert pool.take() == 1 and second.page not in index.by_page and pool.evictions == 1   # the end of the chain first
    pool.hold(0)                                                   # an idle page taken up again keeps its record
    assert pool.refs[0] == 1 and not pool.is_idle(0) and index.by_page[0] is first
    with pytest.raises(CacheFull):
        pool.take()
    pool.let_go(0)
    assert pool.take() == 0 and len(index) == 0


# ----------------------------------------------------------------------------- scenarios
def test_pages_come_back_and_are_used_again():
    m, s = make(pages=4, caching=False)
    for i in range(5):                                         # 5 x 3 pages through a pool of 4
        run(m, s, i, list(range(10 * i, 10 * i + 10)))
        assert m.available_pages() == (1,)
        m.release(i)
        check_invariants(m, s)
        assert m.available_pages() == (4,) and m.stats().pages_in_use == 0


def test_prefix_hit_attaches_whole_pages_and_copies_a_partial_one():
    m, s = make(pages=10)
    first = [1, 2, 3, 4, 5, 6, 7, 8, 9, 10]
    run(m, s, "a", first)
    m.release("a")                                             # 2 full pages + a partial tail stay cached
    cost = m.admission_cost([1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11])
    assert cost.prefill_tokens == 1                            # all ten cached (the tail page whole)
    assert m.admit("b", [1, 2, 3, 4, 5, 6, 77, 78])
    assert m.committed_tokens("b") == 6 and m.counters.partial_copies == 1    # 4 whole + 2 copied
    s.run_step(m, "b")
    m.commit("b", 2)
    check_invariants(m, s)


def test_fork_shares_pages_and_copies_on_write():
    m, s = make(pages=6, caching=False)
    run(m, s, "p", [1, 2, 3, 4, 5, 6])
    m.fork("p", "c")
    check_invariants(m, s)
    assert m.block_table("p") == m.block_table("c") and m.available_pages() == (4,)
    assert m.pages_needed_to_extend("c", 1) == (1,)            # the shared, partly filled page is copied
    decode(m, s, "c", 70)
    decode(m, s, "p", 80)                                      # p is the sole holder again: writes in place
    assert m.counters.cow_copies == 1
    assert m.block_table("p")[0] == m.block_table("c")[0] and m.block_table("p")[1] != m.block_table("c")[1]
    m.release("p"), m.release("c")
    check_invariants(m, s)
    assert m.available_pages() == (6,)


def test_identical_pages_are_deduplicated_at_commit():
    m, s = make(pages=8)
    assert m.admit("a", [1, 2, 3, 4, 5]) and m.admit("b", [1, 2, 3, 4, 6])    # same first page, both computed
    for name in ("a", "b"):
        s.run_step(m, name)
        m.commit(name, 5)
    check_invariants(m, s)
    assert m.counters.dedupes == 1 and m.block_table("a")[0] == m.block_table("b")[0]


def test_eviction_takes_the_least_recently_released_leaf():
    m, s = make(pages=4)
    run(m, s, "a", [1, 2, 3, 4, 5, 6, 7, 8, 9])                # pages: [1234] [5678] [9]
    m.release("a")
    run(m, s, "b", [50, 51, 52, 53, 54])                       # takes the free page, then evicts the tail [9]
    assert m.stats().evictions == 1
    assert m.admission_cost([1, 2, 3, 4, 5, 6, 7, 8, 9, 10]).prefill_tokens == 2    # [9] is gone, 8 remain
    m.release("b")
    check_invariants(m, s)


def test_admit_is_all_or_nothing():
    m, s = make(pages=3, caching=False)
    run(m, s, "a", [1, 2, 3, 4, 5])
    before = (m.available_pages(), dict(m.seqs))
    assert not m.admit("b", list(range(9)))
    assert (m.available_pages(), dict(m.seqs)) == before
    with pytest.raises(CacheFull):
        m.extend("a", list(range(20)))


def test_window_group_gives_pages_back_as_the_window_passes():
    m, s = make(pages=4, windows=(6,), caching=True)           # a window turns prefix reuse off
    assert not m.caching
    run(m, s, "w", list(range(30)), chunk=3)                   # 30 tokens through 4 pages of 4
    assert m.counters.window_releases > 0
    assert m.block_table("w").count(-1) >= 5
    m.release("w")
    check_invariants(m, s)
    assert m.available_pages() == (4,)


def test_two_groups_have_pages_of_their_own():
    m, s = make(pages=8, windows=(0, 5))
    run(m, s, "x", list(range(20)), chunk=4)
    assert m.available_pages()[0] == 3 and m.available_pages()[1] >= 5
    m.fork("x", "y")
    decode(m, s, "y", 99)
    m.release("x"), m.release("y")
    check_invariants(m, s)
    assert m.available_pages() == (8, 8)


def test_groups_that_keep_all_keys_share_one_pool_and_prefix_reuse_survives():
    m, s = make(pages=10, windows=(0, 0))                      # two layer groups of full attention
    assert m.caching and len(m.pools) == 1 and m.pool_of_group == [0, 0]
    run(m, s, "a", [1, 2, 3, 4, 5, 6, 7, 8, 9, 10])
    m.release("a")
    assert m.admit("b", [1, 2, 3, 4, 5, 6, 77])
    assert m.committed_tokens("b") == 6 and m.counters.partial_copies == 1
    assert sorted(c[0] for c in s.copies) == [0, 1]            # the copied run is copied in both groups' tensors
    s.run_step(m, "b")
    m.commit("b", 1)
    check_invariants(m, s)
    m.fork("b", "c")
    decode(m, s, "c", 5)                                       # copy on write, again in both groups
    assert sorted(c[0] for c in s.copies) == [0, 0, 1, 1] and m.block_table("c", 0) == m.block_table("c", 1)


def test_state_slots_are_taken_copied_and_given_back():
    m, s = make(pages=8, caching=True, state_bytes=64, slots=2)
    assert not m.caching                                       # state cannot be rebuilt from cached pages
    run(m, s, "a", [1, 2, 3, 4, 5], chunk=2)
    m.fork("a", "b")
    assert m.state_slot("a") != m.state_slot("b") and s.state[m.state_slot("b")] == [1, 2, 3, 4, 5]
    assert not m.can_fork() and not m.admit("c", [1])          # both slots are taken
    decode(m, s, "b", 9)
    m.release("a")
    assert m.admit("c", [7, 8])
    assert s.state[m.state_slot("c")] == []                    # a reused slot starts cleared
    s.run_step(m, "c"), m.commit("c", 2)
    check_invariants(m, s)


def test_rollback_drops_rejected_slots():
    m, s = make(pages=4, caching=False)
    run(m, s, "a", [1, 2, 3])
    m.extend("a", [4, 5, 6, 7])                                # four candidates
    s.run_step(m, "a")
    m.commit("a", 1)                                           # only one accepted
    check_invariants(m, s)
    assert m.committed_tokens("a") == 4 and len(m.block_table("a")) == 1


def test_layout_groups_entries_by_geometry():
    needs = [(KVNeed(2, 16, 0), 0), (KVNeed(2, 16, 8), 0), (KVNeed(2, 16, 0), 100), (None, 30), (KVNeed(4, 16, 0), 0)]
    layout = plan_layout(needs, 16)
    assert [g.entries for g in layout.groups] == [(0, 2), (1,), (4,)]
    assert layout.state_offsets == (-1, -1, 0, 256, -1) and layout.state_bytes == 512
    assert layout.group_of(2) == (0, 1) and not layout.prefix_reuse_possible
    assert plan_layout(needs[:1], 16).prefix_reuse_possible


# ----------------------------------------------------------------------------- random workloads
@pytest.mark.parametrize("seed", range(12))
@pytest.mark.parametrize("kind", ["cached", "plain", "window", "state", "two_full"])
def test_random_orders_of_requests_keep_the_contract(seed, kind):
    rng = random.Random(1000 * seed + len(kind))
    kwargs = {"cached": {}, "plain": {"caching": False}, "window": {"windows": (0, 7)},
              "state": {"state_bytes": 8, "slots": 5}, "two_full": {"windows": (0, 0)}}[kind]
    m, s = make(pages=rng.choice([6, 9, 14]), page_tokens=rng.choice([2, 4]), **kwargs)
    stems = [[rng.randrange(4) for _ in range(12)] for _ in range(3)]       # shared prefixes are likely
    live, next_id = {}, 0
    for _ in range(250):
        op = rng.random()
        if op < 0.3 or not live:
            stem = rng.choice(stems)
            tokens = stem[:rng.randrange(0, 12)] + [rng.randrange(6) for _ in range(rng.randrange(1, 8))]
            chunk = rng.choice([None, 1, 2, 5])
            if m.admit(next_id, tokens, chunk):
                live[next_id] = list(tokens)
                s.run_step(m, next_id)
                m.commit(next_id, m.reserved_tokens(next_id) - m.committed_tokens(next_id))
            next_id += 1
        elif op < 0.75:
            seq_id = rng.choice(list(live))
            tokens = live[seq_id]
            done = m.committed_tokens(seq_id)
            new = tokens[done:done + rng.randrange(1, 5)] if done < len(tokens) else [rng.randrange(6)]
            if m.can_extend(seq_id, len(new)):
                if done >= len(tokens):
                    tokens.extend(new)
                m.extend(seq_id, new)
                s.run_step(m, seq_id)
                accepted = len(new) if (kind == "state" or rng.random() < 0.8) else rng.randrange(0, len(new) + 1)
                m.commit(seq_id, accepted)
                if done >= len(tokens) - len(new):
                    del tokens[done + accepted:]
        elif op < 0.85 and m.can_fork() and m.fits((1,) * len(m.pools)):
            src = rng.choice(list(live))
            m.fork(src, next_id)
            live[next_id] = list(live[src])
            next_id += 1
        else:
            seq_id = rng.choice(list(live))
            m.release(seq_id)
            del live[seq_id]
        check_invariants(m, s)
        # the one-pass count for a batch of single tokens equals the sum of the per-request counts
        each = [m.pages_needed_to_extend(i, 1) for i in live]
        assert m.pages_for_one_more_each(list(live)) == [sum(e[g] for e in each) for g in range(len(m.pools))]
    for seq_id in list(live):
        m.release(seq_id)
    check_invariants(m, s)
    assert m.stats().pages_in_use == 0
    assert all(pool.available() == pool.num_pages for pool in m.pools), "a page was lost"


def test_a_pending_token_is_amended_before_its_commit_and_dropped_with_a_released_request():
    from tinyserve_llm_b200.cache.manager import PENDING_TOKEN
    layout = layout_of(4)
    storage = FakeStorage(layout, [8])
    m = CacheManager(layout, 8, storage, caching=True)
    assert m.admit("a", [1, 2, 3])
    storage.run_step(m, "a")
    m.commit("a", 3)
    m.extend("a", [PENDING_TOKEN])                     # the token is still on the device
    with pytest.raises(AssertionError, match="pending"):
        m.commit("a", 1)
    m.amend_last("a", 9)
    with pytest.raises(AssertionError, match="no pending token"):
        m.amend_last("a", 9)
    storage.run_step(m, "a")
    m.commit("a", 1)                                   # the page is full: published under its real tokens
    check_invariants(m, storage)
    assert m.admission_cost([1, 2, 3, 9, 5]).prefill_tokens == 1
    m.extend("a", [PENDING_TOKEN])
    with pytest.raises(AssertionError, match="commit first"):
        m.release("a")
    m.release("a", drop_reserved=True)                 # the request ended under a step launched ahead
    check_invariants(m, storage)
    assert m.stats().pages_in_use == 0
