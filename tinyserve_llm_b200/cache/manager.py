"""
Host side of the cache: which pages hold which request's keys and values, and which fixed-size
state slot belongs to which request.  No tensor lives here; copies of page contents are asked of a
`storage` object (the device pools in production, a fake in the CPU tests) and are ordered on its
stream.

Pages.  A layer group (the cache entries whose mixers share kv heads, head size and window) has its
own pool of fixed-size pages and, per request, its own block table.  A group that keeps all keys
holds a request's pages until the request is released; a window group gives pages back as soon as
every token in them is further than `window` behind the committed length, and marks them -1 in the
table.  Released pages are reused.

Prefix reuse.  When there is exactly one group, it keeps all keys and nothing needs per-request
state, released pages stay indexed in a prefix tree (cache/prefix_tree.py) until evicted, least
recently released leaf first, and a new request attaches the longest cached prefix token by token:
whole pages by reference, a partly matching page by copying its matching slots.  A request forked
for parallel sampling shares every page; a shared, partly filled last page is copied before it is
written (copy on write).  Behaviour follows tinyserve-llm's manager (kvcache/manager.py:127-321);
what is new here are layer groups, window release, state slots and reservation in portions.

Protocol per request: admit (reserve the first portion) -> step -> commit -> [extend -> step ->
commit]* -> release.  Tables are valid from a reservation to the commit that follows it, and may
change at commit (an identical page already cached replaces the request's own).
"""

from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass, field, replace
from typing import Protocol, Sequence

from tinyserve_llm_b200.cache.prefix_tree import PageNode, PrefixMatch, PrefixTree


@dataclass(frozen=True)
class GroupLayout:
    """Cache entries that share page geometry."""

    entries: tuple[int, ...]          # cache entry ids (ModelSpec.run[*].cache_entry) in this group
    num_kv_heads: int
    head_dim: int
    window: int = 0                   # 0: all keys kept


@dataclass(frozen=True)
class CacheLayout:
    page_tokens: int
    groups: tuple[GroupLayout, ...]
    state_offsets: tuple[int, ...]    # per cache entry: byte offset of its state inside a slot, -1 if none
    state_bytes: int                  # bytes of one request's state slot (0: no entry keeps state)
    state_sizes: tuple[int, ...] = ()  # per cache entry: bytes of its state (0 if none)

    @property
    def prefix_reuse_possible(self) -> bool:
        return len(self.groups) == 1 and self.groups[0].window == 0 and self.state_bytes == 0

    def group_of(self, entry: int) -> tuple[int, int]:
        """(group index, index of the entry inside its group)."""
        for g, group in enumerate(self.groups):
            if entry in group.entries:
                return g, group.entries.index(entry)
        raise KeyError(f"cache entry {entry} keeps no keys and values")


def plan_layout(needs: Sequence[tuple[object | None, int]], page_tokens: int) -> CacheLayout:
    """
    Groups cache entries by what their mixers need.  `needs[e]` is (kv need or None, state bytes) of
    entry e, the kv need having num_kv_heads, head_dim and window attributes.
    """
    if page_tokens <= 0:
        raise ValueError(f"page size must be positive, got {page_tokens}")
    by_geometry: dict[tuple[int, int, int], list[int]] = {}
    offsets, total = [], 0
    sizes = tuple(int(state) for _, state in needs)
    for e, (kv, state) in enumerate(needs):
        if kv is not None:
            by_geometry.setdefault((kv.num_kv_heads, kv.head_dim, kv.window), []).append(e)
        if state > 0:
            offsets.append(total)
            total += -(-state // 256) * 256         # slots of each entry start 256-byte aligned
        else:
            offsets.append(-1)
    groups = tuple(GroupLayout(tuple(es), nkv, hd, w) for (nkv, hd, w), es in by_geometry.items())
    return CacheLayout(page_tokens, groups, tuple(offsets), total, sizes)


class Storage(Protocol):
    """What the manager asks of the device side."""

    def copy_slots(self, group: int, src_page: int, dst_page: int, num_slots: int) -> None: ...
    def copy_state(self, src_slot: int, dst_slot: int) -> None: ...
    def clear_state(self, slot: int) -> None: ...


class NullStorage:
    """Storage that moves nothing: for sizing runs and host-only tests that do not look at contents."""

    def copy_slots(self, group: int, src_page: int, dst_page: int, num_slots: int) -> None:
        pass

    def copy_state(self, src_slot: int, dst_slot: int) -> None:
        pass

    def clear_state(self, slot: int) -> None:
        pass


PENDING_TOKEN = -1      # stands in the token record for a token that is still on the device; amend_last() fills it in


@dataclass
class SeqState:
    tables: list[list[int]]                        # per group, page ids in token order (-1: given back)
    tokens: list[int] = field(default_factory=list)  # one per reserved slot
    committed: int = 0
    state_slot: int = -1

    @property
    def reserved(self) -> int:
        return len(self.tokens)


@dataclass(frozen=True)
class AdmissionCost:
    pages_needed: tuple[int, ...]     # per group, to hold the whole request; compare with available_pages()
    prefill_tokens: int               # tokens the model has to run


@dataclass
class CacheStats:
    """Running totals; `pages_in_use` and `cached_pages` are current values filled in by stats()."""

    evictions: int = 0
    cow_copies: int = 0
    partial_copies: int = 0
    publishes: int = 0
    dedupes: int = 0
    window_releases: int = 0
    pages_in_use: int = 0
    cached_pages: int = 0


class CacheFull(RuntimeError):
    """A reservation was asked for without checking that it fits."""


class _Pool:
    """Reference counts and the free list of one group's pages."""

    def __init__(self, num_pages: int) -> None:
        self.num_pages = num_pages
        self.refs = [0] * num_pages
        self.free = list(range(num_pages - 1, -1, -1))     # pop() hands out page 0 first
        self.free_cached: OrderedDict[int, None] = OrderedDict()   # ref 0 but still in the prefix tree, oldest first

    def available(self) -> int:
        return len(self.free) + len(self.free_cached)


class CacheManager:
    def __init__(self, layout: CacheLayout, num_pages: int | Sequence[int], storage: Storage | None = None, *,
                 caching: bool = True, num_state_slots: int = 0) -> None:
        self.layout = layout
        self.page_tokens = layout.page_tokens
        counts = [num_pages] * len(layout.groups) if isinstance(num_pages, int) else list(num_pages)
        if len(counts) != len(layout.groups) or any(c <= 0 for c in counts):
            raise ValueError(f"need a positive page count per layer group ({len(layout.groups)}), got {counts}")
        self.pools = [_Pool(c) for c in counts]
        self.storage: Storage = storage if storage is not None else NullStorage()
        self.caching = bool(caching) and layout.prefix_reuse_possible
        self.tree = PrefixTree(self.page_tokens)
        self.seqs: dict[int, SeqState] = {}
        self._clock = 0
        self.counters = CacheStats()
        if layout.state_bytes and num_state_slots <= 0:
            raise ValueError("the model keeps per-request state: num_state_slots must be positive")
        self.num_state_slots = num_state_slots
        self._free_slots = list(range(num_state_slots - 1, -1, -1))

    # ------------------------------------------------------------------ queries
    @property
    def num_pages(self) -> int:
        """Pages of the smallest pool: the bound requests are checked against."""
        return min((p.num_pages for p in self.pools), default=1 << 30)

    def available_pages(self) -> tuple[int, ...]:
        return tuple(p.available() for p in self.pools)

    def fits(self, pages: Sequence[int], reserve: int = 0) -> bool:
        return all(need + reserve <= pool.available() for need, pool in zip(pages, self.pools))

    def free_state_slots(self) -> int:
        return len(self._free_slots) if self.layout.state_bytes else 1 << 30

    def block_table(self, seq_id: int, group: int = 0) -> list[int]:
        return self.seqs[seq_id].tables[group]

    def state_slot(self, seq_id: int) -> int:
        return self.seqs[seq_id].state_slot

    def committed_tokens(self, seq_id: int) -> int:
        """Leading tokens whose keys and values are in the cache: where the next portion starts."""
        return self.seqs[seq_id].committed

    def reserved_tokens(self, seq_id: int) -> int:
        return self.seqs[seq_id].reserved

    def stats(self) -> CacheStats:
        in_use = sum(p.num_pages - p.available() for p in self.pools)
        return replace(self.counters, pages_in_use=in_use, cached_pages=len(self.tree.nodes))

    # ------------------------------------------------------------------ page bookkeeping
    def _take(self, g: int) -> int:
        pool = self.pools[g]
        if pool.free:
            page = pool.free.pop()
        else:
            page = self._evict(pool)
        assert pool.refs[page] == 0
        pool.refs[page] = 1
        return page

    def _evict(self, pool: _Pool) -> int:
        # Oldest released first; a free page's descendants are free too and were released before
        # it (tails go first), so the first leaf met is the least recently used one.
        for page in pool.free_cached:
            node = self.tree.nodes[page]
            if not node.children:
                del pool.free_cached[page]
                self.counters.evictions += 1
                return self.tree.evict(node)
        raise CacheFull("no free page: check available_pages() before reserving")

    def _hold(self, g: int, page: int) -> None:
        pool = self.pools[g]
        if pool.refs[page] == 0:
            assert page in pool.free_cached, "a free page that is not cached must be taken, not held"
            del pool.free_cached[page]
        pool.refs[page] += 1

    def _drop(self, g: int, page: int) -> None:
        pool = self.pools[g]
        assert pool.refs[page] > 0, f"page {page} of group {g} is released twice"
        pool.refs[page] -= 1
        if pool.refs[page]:
            return
        node = self.tree.nodes.get(page) if g == 0 else None
        if node is None:
            pool.free.append(page)
        else:
            self._clock += 1
            node.stamp = self._clock
            pool.free_cached[page] = None

    # ------------------------------------------------------------------ admission
    def _source(self, match: PrefixMatch) -> PageNode | None:
        """The page a partial match is copied from: one that is in use if there is one (it cannot be evicted)."""
        if not match.partial_len:
            return None
        refs = self.pools[0].refs
        return min(match.partial_sources, key=lambda p: (refs[p.page] == 0, p.page))

    def _match(self, tokens: Sequence[int], reuse_limit: int | None = None) -> PrefixMatch:
        if not self.caching:
            return PrefixMatch([])
        if reuse_limit is not None and reuse_limit < len(tokens) - 1:
            tokens = tokens[:max(reuse_limit, 0) + 1]      # the walk stops one token short of what it is given
        return self.tree.match(tokens)

    def _cost(self, match: PrefixMatch, source: PageNode | None, num_tokens: int,
              max_new: int | None = None) -> AdmissionCost:
        B = self.page_tokens
        whole = -(-num_tokens // B)
        first = num_tokens if max_new is None else min(num_tokens, match.num_tokens + max_new)
        costs = []
        for g, group in enumerate(self.layout.groups):
            if g == 0 and self.caching:
                refs = self.pools[0].refs
                need = whole - len(match.pages)
                last = match.pages[-1] if match.pages else None
                if last is not None and len(last.tokens) < B and refs[last.page] > 0:
                    need += 1                          # an attached, shared, partly filled page is copied on write
                if source is not None and refs[source.page] == 0:
                    need = max(need, 2)                # a free source must survive until its copy is made
                need += sum(1 for p in match.pages if refs[p.page] == 0)   # attached free pages leave the pool
                costs.append(need)
            elif group.window:
                costs.append(-(-first // B))           # a window group needs the first portion's pages only
            else:
                costs.append(whole)
        return AdmissionCost(tuple(costs), num_tokens - match.num_tokens)

    def admission_cost(self, tokens: Sequence[int], max_new: int | None = None,
                       reuse_limit: int | None = None) -> AdmissionCost:
        """What admitting these tokens would take from the pools and how many tokens it would run.  Read-only."""
        match = self._match(tokens, reuse_limit)
        return self._cost(match, self._source(match), len(tokens), max_new)

    def admit(self, seq_id: int, tokens: Sequence[int], max_new: int | None = None,
              reuse_limit: int | None = None) -> bool:
        """
        Starts a request: attaches its cached prefix, copies a partial match, takes a state slot and
        reserves slots for the next `max_new` tokens after the prefix (None: all the rest).  Returns
        False, changing nothing, if the pools cannot hold the whole request right now.
        `reuse_limit`: at most this many leading tokens are taken from the cache (a caller that
        wants the model's output at a prompt position must have that position run).
        """
        assert len(tokens) > 0, "a request needs at least one token"
        assert seq_id not in self.seqs, "the request is admitted already"
        match = self._match(tokens, reuse_limit)
        source = self._source(match)
        if not self.fits(self._cost(match, source, len(tokens), max_new).pages_needed):
            return False
        if self.layout.state_bytes and not self._free_slots:
            return False
        seq = SeqState(tables=[[] for _ in self.pools])
        for node in match.pages:                       # hold matched pages before anything is taken: no eviction
            self._hold(0, node.page)
            seq.tables[0].append(node.page)
        if source is not None:
            self._hold(0, source.page)
            dst = self._take(0)
            self.storage.copy_slots(0, source.page, dst, match.partial_len)
            self.counters.partial_copies += 1
            self._drop(0, source.page)                 # the copy is ordered on the stream before any reuse
            seq.tables[0].append(dst)
        seq.committed = match.num_tokens
        seq.tokens = list(tokens[:seq.committed])
        if self.layout.state_bytes:
            seq.state_slot = self._free_slots.pop()
            self.storage.clear_state(seq.state_slot)
        rest = tokens[seq.committed:]
        if max_new is not None:
            rest = rest[:max_new]
        self.seqs[seq_id] = seq
        self._reserve(seq, rest)
        return True

    # ------------------------------------------------------------------ reservation
    def _pages_to_reserve(self, seq: SeqState, n: int) -> tuple[int, ...]:
        B = self.page_tokens
        out = []
        for g, pool in enumerate(self.pools):
            table = seq.tables[g]
            need = -(-(seq.reserved + n) // B) - len(table)
            if seq.reserved % B and table and table[-1] >= 0 and pool.refs[table[-1]] > 1:
                need += 1                              # the shared last page is copied before the write
            out.append(max(need, 0))
        return tuple(out)

    def pages_needed_to_extend(self, seq_id: int, n: int) -> tuple[int, ...]:
        return self._pages_to_reserve(self.seqs[seq_id], n)

    def can_extend(self, seq_id: int, n: int) -> bool:
        return self.fits(self.pages_needed_to_extend(seq_id, n))

    def pages_for_one_more_each(self, seq_ids: Sequence) -> list[int]:
        """Per group, the pages that one more token for each of these requests would take: one pass, for large batches."""
        B = self.page_tokens
        need = [0] * len(self.pools)
        seqs = self.seqs
        for seq_id in seq_ids:
            seq = seqs[seq_id]
            reserved = len(seq.tokens)
            whole = reserved // B + 1
            inside = reserved % B
            for g, pool in enumerate(self.pools):
                table = seq.tables[g]
                if whole > len(table):
                    need[g] += whole - len(table)
                if inside and table and table[-1] >= 0 and pool.refs[table[-1]] > 1:
                    need[g] += 1                       # the shared last page is copied before the write
        return need

    def extend(self, seq_id: int, tokens: Sequence[int], checked: bool = False) -> None:
        """
        Reserves slots for the step's tokens of a running request; commit() closes the step.
        `checked`: the caller has made sure the pages are there (pages_for_one_more_each + fits).
        """
        assert len(tokens) > 0, "a step feeds at least one token"
        seq = self.seqs[seq_id]
        assert len(seq.tokens) == seq.committed, "the previous step was not committed"
        if not checked and not self.fits(self._pages_to_reserve(seq, len(tokens))):
            raise CacheFull("not enough free pages: check can_extend() first")
        self._reserve(seq, tokens)

    def _reserve(self, seq: SeqState, tokens: Sequence[int]) -> None:
        B = self.page_tokens
        used = seq.reserved % B
        for g, pool in enumerate(self.pools):
            table = seq.tables[g]
            if used and table and table[-1] >= 0:
                last = table[-1]
                if pool.refs[last] > 1:                # shared: copy on write
                    fresh = self._take(g)
                    self.storage.copy_slots(g, last, fresh, used)
                    self.counters.cow_copies += 1
                    self._drop(g, last)
                    table[-1] = fresh
                else:
                    node = self.tree.nodes.get(last) if g == 0 else None
                    assert node is None or used >= len(node.tokens), "a published slot would be overwritten"
            want = -(-(seq.reserved + len(tokens)) // B)
            while len(table) < want:
                table.append(self._take(g))
        seq.tokens.extend(tokens)

    # ------------------------------------------------------------------ commit / release / fork
    def commit(self, seq_id: int, num_accepted: int) -> None:
        """
        Closes a step: keeps the first `num_accepted` slots reserved since the last commit, drops the
        rest, publishes pages that became full, and gives back pages a window has passed.
        """
        seq = self.seqs[seq_id]
        assert 0 <= num_accepted <= seq.reserved - seq.committed, "more slots accepted than reserved"
        assert not self.layout.state_bytes or num_accepted == seq.reserved - seq.committed, \
            "a model with per-request state cannot take back tokens it has run"
        assert PENDING_TOKEN not in seq.tokens[seq.committed:seq.committed + num_accepted], \
            "a token still pending would be committed: amend it first"
        B = self.page_tokens
        before = seq.committed
        seq.committed += num_accepted
        del seq.tokens[seq.committed:]
        keep = -(-seq.committed // B)
        for g in range(len(self.pools)):
            table = seq.tables[g]
            while len(table) > keep:
                page = table.pop()
                if page >= 0:
                    self._drop(g, page)
        if self.caching:
            for i in range(before // B, seq.committed // B):
                self._publish(seq, i)
        for g, group in enumerate(self.layout.groups):
            if group.window:
                self._release_behind_window(seq, g, group.window)

    def _release_behind_window(self, seq: SeqState, g: int, window: int) -> None:
        # The next query sits at position `committed` and sees keys >= committed - window + 1.
        first_needed = max(0, seq.committed - window + 1)
        table = seq.tables[g]
        for i in range(min(first_needed // self.page_tokens, len(table))):
            if table[i] >= 0:
                self._drop(g, table[i])
                table[i] = -1
                self.counters.window_releases += 1

    def _publish(self, seq: SeqState, i: int) -> None:
        B = self.page_tokens
        table = seq.tables[0]
        page = table[i]
        parent = self.tree.nodes[table[i - 1]] if i else self.tree.root
        tokens = seq.tokens[i * B:min((i + 1) * B, seq.committed)]
        node = self.tree.nodes.get(page)
        if node is None:
            kept = self.tree.publish(parent, page, tokens)
            if kept.page == page:
                self.counters.publishes += 1
        elif len(node.tokens) < len(tokens):
            assert node.parent is parent
            kept = self.tree.grow(node, tokens)
        else:
            return
        if kept.page != page:                          # the same tokens are cached already: use that page
            self.counters.dedupes += 1
            self._hold(0, kept.page)
            table[i] = kept.page
            self._drop(0, page)

    def amend_last(self, seq_id: int, token: int) -> None:
        """Fills in the one reserved token that was extended as PENDING_TOKEN, before its commit."""
        seq = self.seqs[seq_id]
        assert seq.reserved == seq.committed + 1 and seq.tokens[-1] == PENDING_TOKEN, "no pending token to amend"
        seq.tokens[-1] = token

    def release(self, seq_id: int, drop_reserved: bool = False) -> None:
        """
        Ends a request (finished or preempted).  With prefix reuse its pages stay cached until evicted.
        `drop_reserved`: slots reserved for a step that will not be committed go with it (a request
        that ended while its next step was already launched).
        """
        seq = self.seqs[seq_id]
        assert drop_reserved or seq.reserved == seq.committed, "release between steps: commit first"
        del seq.tokens[seq.committed:]
        if self.caching and seq.committed % self.page_tokens:
            self._publish(seq, seq.committed // self.page_tokens)
        del self.seqs[seq_id]
        for g in range(len(self.pools)):
            for page in reversed(seq.tables[g]):       # tail first: leaves get older stamps than their parents
                if page >= 0:
                    self._drop(g, page)
        if seq.state_slot >= 0:
            self._free_slots.append(seq.state_slot)

    def can_fork(self) -> bool:
        return not self.layout.state_bytes or bool(self._free_slots)

    def fork(self, src_id: int, new_id: int) -> None:
        """Starts `new_id` as a copy of `src_id` sharing all its pages; its state slot is copied."""
        assert new_id not in self.seqs, "the request is admitted already"
        src = self.seqs[src_id]
        assert src.reserved == src.committed, "fork between steps: commit first"
        slot = -1
        if self.layout.state_bytes:
            if not self._free_slots:
                raise CacheFull("no free state slot: check can_fork() first")
            slot = self._free_slots.pop()
            self.storage.copy_state(src.state_slot, slot)
        for g in range(len(self.pools)):
            for page in src.tables[g]:
                if page >= 0:
                    self._hold(g, page)
        self.seqs[new_id] = SeqState(tables=[list(t) for t in src.tables], tokens=list(src.tokens),
                                     committed=src.committed, state_slot=slot)
