"""The replay for cached paths, on the host alone: the trace the GPU test replays does take every path it is meant to."""

import pytest

import replay_util as ru
from tiny_configs import PAGE_A, PAGE_B, TINY_A, TINY_B


@pytest.mark.parametrize("raw, page", [(TINY_A, PAGE_A), (TINY_B, PAGE_B)], ids=["a", "b"])
def test_the_cached_paths_trace_takes_every_path(raw, page):
    trace, requests = ru.cached_paths_trace(raw["vocab_size"], page)
    pages = ru.smallest_pool(trace, caching=True) + 4
    stats, reused = ru.simulate(trace, pages, caching=True)
    shared = 6 * page + page // 4
    assert reused["q"] == shared                               # six pages attached and a quarter page copied
    assert stats.partial_copies >= 1 and stats.cow_copies >= 1 and stats.dedupes >= 3 and stats.evictions > 0
    assert 0 < reused["p_again"] < len(requests["p"]) - 1      # part of P survived, part was evicted and is run again
    assert reused["r3"] == 0                                   # its first row is wanted: everything runs
    assert pages * page < sum(-(-len(v) // page) * page for v in requests.values()), "pages must be used again"
    assert stats.pages_in_use == 0
    assert max(len(v) for v in requests.values()) <= raw["max_position_embeddings"]


def test_without_caching_the_same_trace_reuses_nothing_but_still_forks():
    trace, _ = ru.cached_paths_trace(TINY_A["vocab_size"], PAGE_A)
    stats, reused = ru.simulate(trace, ru.smallest_pool(trace, caching=False), caching=False)
    assert not any(reused.values()) and stats.cow_copies == 1 and stats.publishes == 0 and stats.dedupes == 0
