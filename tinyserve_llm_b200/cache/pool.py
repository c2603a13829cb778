"""
One pool of pages: who holds how many references, which pages are blank, and which cached pages
nobody holds (they stay readable until their page is needed for something else).

A page is in exactly one of three states: held (reference count above zero), blank (free, holds
nothing on record) or idle (free, still on record in the pool's `PrefixIndex`).  Blank pages are
handed out first; when there are none the idle page goes that was let go of longest ago among
those no other cached page continues from (its keys cannot be reached without it).  Candidates
wait in a heap ordered by the time they became idle; an entry is checked when it comes up and
thrown away if the page was taken up again meanwhile, so holding and letting go cost O(log n) and
nothing is ever scanned.  (tinyserve-llm scans all cached pages for the oldest free leaf,
kvcache/manager.py:85-98; the order of eviction is the same.)
"""

from __future__ import annotations

import heapq

from tinyserve_llm_b200.cache.prefix_index import CachedPage, PrefixIndex


class CacheFull(RuntimeError):
    """A page was asked for without checking that one is available."""


class PagePool:
    def __init__(self, num_pages: int, index: PrefixIndex | None = None) -> None:
        self.num_pages = num_pages
        self.index = index                                 # None: nothing of this pool is ever on record
        self.refs = [0] * num_pages
        self._blank = list(range(num_pages - 1, -1, -1))  # a stack: page 0 goes out first
        self._idle: dict[int, int] = {}                    # idle page -> when it became idle
        self._oldest: list[tuple[int, int]] = []           # (when, page) of idle pages nothing continues from; may be stale
        self._clock = 0
        self.evictions = 0

    # ------------------------------------------------------------------ queries
    def available(self) -> int:
        return len(self._blank) + len(self._idle)

    def in_use(self) -> int:
        return self.num_pages - self.available()

    def is_idle(self, page: int) -> bool:
        return page in self._idle

    def blank_pages(self) -> list[int]:
        return list(self._blank)

    def idle_pages(self) -> list[int]:
        return list(self._idle)

    def cached(self, page: int) -> CachedPage | None:
        return self.index.by_page.get(page) if self.index is not None else None

    # ------------------------------------------------------------------ references
    def take(self) -> int:
        """A page to write into, held once: a blank one, else the stalest idle page, which goes off the record."""
        page = self._blank.pop() if self._blank else self._evict()
        assert self.refs[page] == 0
        self.refs[page] = 1
        return page

    def hold(self, page: int) -> None:
        """One more reference; an idle page comes back into use with its contents."""
        if self.refs[page] == 0:
            assert page in self._idle, "a free page without a record is taken, not held"
            del self._idle[page]                           # its heap entry, if any, is stale from now on
        self.refs[page] += 1

    def let_go(self, page: int) -> None:
        """One reference less; the last one leaves the page blank, or idle if it is on record."""
        assert self.refs[page] > 0, f"page {page} is let go of twice"
        self.refs[page] -= 1
        if self.refs[page]:
            return
        entry = self.cached(page)
        if entry is None:
            self._blank.append(page)
            return
        self._clock += 1
        entry.idle_since = self._idle[page] = self._clock
        if not entry.after:
            heapq.heappush(self._oldest, (self._clock, page))

    def _evict(self) -> int:
        while self._oldest:
            when, page = heapq.heappop(self._oldest)
            if self._idle.get(page) != when:
                continue                                   # taken up again since, or gone already
            entry = self.index.by_page[page]
            if entry.after:
                continue                                   # a page was filed behind it meanwhile
            before = entry.before
            self.index.drop(entry)
            del self._idle[page]
            self.evictions += 1
            # the page before it may now be the end of its chain: if it is idle too, it joins the candidates
            if before.page >= 0 and not before.after and before.page in self._idle:
                heapq.heappush(self._oldest, (self._idle[before.page], before.page))
            return page
        raise CacheFull("no free page: check available_pages() before reserving")
