"""
Index of cached pages by the tokens they hold: which pages a new request may take over instead of
computing their keys and values again.

Every cached page hangs under the page that holds the tokens before it (the first page of a
request under the root) and records the tokens whose keys and values it holds; a page that is full
may have pages after it, a partly filled one is always a leaf.  The pages after one page are kept
in ONE list sorted by their tokens, and that list is all there is to search: a run of tokens that
several pages begin with lies in it side by side, so the page that shares the longest run with a
prompt is a neighbour of the place where the prompt's own tokens would be inserted.  One bisection
and a look to both sides answer "is this exact page cached" and "which cached page starts with
most of these tokens" alike; there is no separate table of whole pages and no trie.

What is reused follows tinyserve-llm (kvcache/page_tree.py:43-70): a prompt takes over cached pages
from its first token on, whole pages by reference, and of the first page that does not match as a
whole the tokens it begins with (by a copy the caller makes); the prompt's last token is never
taken from the cache, so that a request always has a token to run.
"""

from __future__ import annotations

from bisect import bisect_left
from operator import attrgetter
from typing import Iterable, Sequence

_tokens_of = attrgetter("tokens")


def shared_run(a: tuple, b: tuple) -> int:
    """How many leading tokens two runs share; whole slices are compared, so equal stretches cost one comparison."""
    n = min(len(a), len(b))
    if a[:n] == b[:n]:
        return n
    low, high = 0, n                            # a[:low] == b[:low], a[:high] != b[:high]
    while high - low > 1:
        mid = (low + high) // 2
        if a[low:mid] == b[low:mid]:
            low = mid
        else:
            high = mid
    return low


class CachedPage:
    """A page of the pool whose contents are on record."""

    __slots__ = ("page", "tokens", "before", "after", "idle_since")

    def __init__(self, page: int, tokens: tuple[int, ...], before: "CachedPage | None") -> None:
        self.page = page                        # id in the pool; -1 for the root, which is no page
        self.tokens = tokens                    # the tokens whose keys and values it holds; grows while its writer fills it
        self.before = before                    # the page holding the tokens before these
        self.after: list[CachedPage] = []       # the pages that continue from here, sorted by their tokens
        self.idle_since = 0                     # when its last holder let go of it (the pool's clock)

    def is_full(self, page_tokens: int) -> bool:
        return len(self.tokens) == page_tokens


class Reuse:
    """What a prompt can take from the cache."""

    __slots__ = ("pages", "run", "starting_with_run")

    def __init__(self, pages: list[CachedPage], run: int = 0, starting_with_run: Sequence[CachedPage] = ()) -> None:
        self.pages = pages                          # taken over as they are, in order
        self.run = run                              # tokens more, which the pages in `starting_with_run` begin with
        self.starting_with_run = list(starting_with_run)

    @property
    def num_tokens(self) -> int:
        return sum(len(p.tokens) for p in self.pages) + self.run


class PrefixIndex:
    def __init__(self, page_tokens: int) -> None:
        self.page_tokens = page_tokens
        self.root = CachedPage(-1, (), None)
        self.by_page: dict[int, CachedPage] = {}

    def __len__(self) -> int:
        return len(self.by_page)

    # ------------------------------------------------------------------ searching
    @staticmethod
    def _position(under: CachedPage, tokens: tuple[int, ...]) -> int:
        return bisect_left(under.after, tokens, key=_tokens_of)

    def _exact(self, under: CachedPage, tokens: tuple[int, ...]) -> CachedPage | None:
        i = self._position(under, tokens)
        if i < len(under.after) and under.after[i].tokens == tokens:
            return under.after[i]
        return None

    def nearest(self, under: CachedPage, tokens: tuple[int, ...]) -> tuple[int, list[CachedPage]]:
        """
        (n, pages): the longest run of leading tokens that `tokens` shares with a page after
        `under`, and all pages after `under` that begin with that run (none if n is 0).
        In a sorted list the shared run can only shrink with the distance from the place where
        `tokens` would stand, so the search walks outwards from there and stops at the first
        page on each side that shares less.
        """
        after = under.after
        if not after or not tokens:
            return 0, []
        here = self._position(under, tokens)
        best = 0
        for i in (here - 1, here):
            if 0 <= i < len(after):
                best = max(best, shared_run(tokens, after[i].tokens))
        if best == 0:
            return 0, []
        sharing = []
        i = here - 1
        while i >= 0 and shared_run(tokens, after[i].tokens) == best:
            sharing.append(after[i])
            i -= 1
        i = here
        while i < len(after) and shared_run(tokens, after[i].tokens) == best:
            sharing.append(after[i])
            i += 1
        return best, sharing

    def lookup(self, tokens: Sequence[int], limit: int | None = None) -> Reuse:
        """
        The cached start of `tokens`, at most `limit` tokens of it and never the last token.
        Page by page: the next stretch of the prompt (up to a page) is looked for among the pages
        after the last one taken.  A page that holds exactly a leading part of the stretch is taken
        whole (and the walk goes on behind it if it is full); otherwise the pages that share most
        with the stretch are reported, for a copy of that run.
        """
        most = len(tokens) - 1
        if limit is not None:
            most = min(most, max(limit, 0))
        taken: list[CachedPage] = []
        under, at = self.root, 0
        while at < most:
            stretch = tuple(tokens[at:min(at + self.page_tokens, most)])
            run, sharing = self.nearest(under, stretch)
            if run == 0:
                break
            whole = next((p for p in sharing if len(p.tokens) == run), None)
            if whole is None:
                return Reuse(taken, run, sharing)
            taken.append(whole)
            at += run
            if not whole.is_full(self.page_tokens):
                break
            under = whole
        return Reuse(taken)

    # ------------------------------------------------------------------ changing
    def file(self, under: CachedPage, page: int, tokens: Iterable[int]) -> CachedPage:
        """
        Puts `page`, which holds `tokens`, on record behind `under`.  If a page with exactly these
        tokens is on record there already, nothing changes and that page is returned: the caller
        has computed the same page twice and keeps one.
        """
        tokens = tuple(tokens)
        assert 0 < len(tokens) <= self.page_tokens, "a page holds between one token and a page of them"
        assert under is self.root or under.is_full(self.page_tokens), "only a full page is continued"
        assert page not in self.by_page, "the page is on record already; lengthen it"
        i = self._position(under, tokens)
        if i < len(under.after) and under.after[i].tokens == tokens:
            return under.after[i]
        entry = CachedPage(page, tokens, under)
        under.after.insert(i, entry)
        self.by_page[page] = entry
        return entry

    def lengthen(self, entry: CachedPage, tokens: Iterable[int]) -> CachedPage:
        """
        The writer of a partly filled page has added tokens to it.  Returns the entry under its
        longer tokens, or, unchanged, the page beside it that holds exactly these tokens already.
        """
        tokens = tuple(tokens)
        old = entry.tokens
        assert len(old) < len(tokens) <= self.page_tokens and tokens[:len(old)] == old, "a page only gains tokens"
        under = entry.before
        twin = self._exact(under, tokens)
        if twin is not None:
            return twin
        del under.after[self._index_of(entry)]
        entry.tokens = tokens
        under.after.insert(self._position(under, tokens), entry)
        return entry

    def drop(self, entry: CachedPage) -> None:
        """Takes a page off the record; only a page nothing continues from may go."""
        assert not entry.after, "a page that others continue from stays on record"
        del entry.before.after[self._index_of(entry)]
        del self.by_page[entry.page]

    def _index_of(self, entry: CachedPage) -> int:
        siblings = entry.before.after
        i = self._position(entry.before, entry.tokens)
        assert i < len(siblings) and siblings[i] is entry, "the record is out of order"
        return i
