"""
Host side of the cache: which pages hold which request's keys and values, and which fixed-size
state slot belongs to which request.  No tensor lives here; copies of page contents are asked of a
`storage` object (the device pools in production, a fake in the CPU tests) and are ordered on its
stream.

Pools.  Layer groups (the cache entries whose mixers share kv heads, head size and window) that
keep all keys fill and empty in step with one another, so they share ONE pool of page ids and one
block table per request: page p of a request is page p in each of these groups' tensors.  Every
group with a window has a pool and a table of its own: it gives a page back as soon as every token
in it is further than `window` behind the committed length, and marks it -1 in the table.

Prefix reuse (where no group has a window and nothing needs per-request state).  What a request
has committed goes on record, page by page, in the shared pool's `PrefixIndex`; the pages stay
readable after the request has gone, until the pool needs them (`PagePool`: the page let go of
longest ago that no other page continues from goes first).  A new request takes over the longest
recorded start of its tokens: whole pages by reference, and of the next page the slots it begins
with, by a copy.  A request forked for parallel sampling shares every page; whoever writes first
into a shared, partly filled page gets a copy of its own (copy on write).  What is reused, when
pages are shared, copied and given back follows tinyserve-llm's manager (kvcache/manager.py:127-321);
the pools, the window release, state slots, reservation in portions, the admission plan and the
index are this engine's own.

Protocol per request: admit (reserve the first portion) -> step -> commit -> [extend -> step ->
commit]* -> release.  Tables are valid from a reservation to the commit that follows it, and may
change at commit (an identical page already on record replaces the request's own).
"""

from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Protocol, Sequence

from tinyserve_llm_b200.cache.pool import CacheFull, PagePool
from tinyserve_llm_b200.cache.prefix_index import CachedPage, PrefixIndex, Reuse


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
        """Cached pages can stand in for a prompt's start only if every layer keeps all keys and none keeps state."""
        return bool(self.groups) and all(g.window == 0 for g in self.groups) and self.state_bytes == 0

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
    tables: list[list[int]]                        # per pool, page ids in token order (-1: given back)
    tokens: list[int] = field(default_factory=list)  # one per reserved slot
    committed: int = 0
    state_slot: int = -1

    @property
    def reserved(self) -> int:
        return len(self.tokens)


@dataclass(frozen=True)
class AdmissionCost:
    pages_needed: tuple[int, ...]     # per pool, to hold the whole request; compare with available_pages()
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


@dataclass
class _Admission:
    """How a request would start: worked out once, priced by `admission_cost`, carried out by `admit`."""

    reuse: Reuse                      # what the index offers
    copy_from: CachedPage | None      # the page whose leading `reuse.run` slots are copied
    reserve: int                      # tokens reserved right away, after the reused ones
    demand: tuple[int, ...]           # pages each pool must have available (the largest need on the way, not the sum)
    prefill_tokens: int


class CacheManager:
    def __init__(self, layout: CacheLayout, num_pages: int | Sequence[int], storage: Storage | None = None, *,
                 caching: bool = True, num_state_slots: int = 0) -> None:
        self.layout = layout
        self.page_tokens = layout.page_tokens
        counts = [num_pages] * len(layout.groups) if isinstance(num_pages, int) else list(num_pages)
        if len(counts) != len(layout.groups) or any(c <= 0 for c in counts):
            raise ValueError(f"need a positive page count per layer group ({len(layout.groups)}), got {counts}")
        self.storage: Storage = storage if storage is not None else NullStorage()
        self.caching = bool(caching) and layout.prefix_reuse_possible
        # groups that keep all keys share the first pool made for one of them; a window group gets its own
        self.pools: list[PagePool] = []
        self.pool_of_group: list[int] = []
        self.groups_of_pool: list[list[int]] = []
        self.window_of_pool: list[int] = []
        shared = -1
        for g, (group, count) in enumerate(zip(layout.groups, counts)):
            if group.window == 0 and shared >= 0:
                self.pool_of_group.append(shared)
                self.groups_of_pool[shared].append(g)
                continue
            if group.window == 0:
                shared = len(self.pools)
                count = min(c for c, other in zip(counts, layout.groups) if other.window == 0)
            self.pool_of_group.append(len(self.pools))
            self.groups_of_pool.append([g])
            self.window_of_pool.append(group.window)
            self.pools.append(PagePool(count))
        self.shared = shared                               # index of the pool of the keep-all groups, -1 if there is none
        self.index: PrefixIndex | None = None
        if self.caching:
            self.index = self.pools[shared].index = PrefixIndex(self.page_tokens)
        self.seqs: dict[int, SeqState] = {}
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
        return self.seqs[seq_id].tables[self.pool_of_group[group]]

    def state_slot(self, seq_id: int) -> int:
        return self.seqs[seq_id].state_slot

    def committed_tokens(self, seq_id: int) -> int:
        """Leading tokens whose keys and values are in the cache: where the next portion starts."""
        return self.seqs[seq_id].committed

    def reserved_tokens(self, seq_id: int) -> int:
        return self.seqs[seq_id].reserved

    def stats(self) -> CacheStats:
        return replace(self.counters, evictions=sum(p.evictions for p in self.pools),
                       pages_in_use=sum(p.in_use() for p in self.pools),
                       cached_pages=len(self.index) if self.index is not None else 0)

    def _copy(self, pool: int, src: int, dst: int, slots: int) -> None:
        for g in self.groups_of_pool[pool]:                # the same page id in every group of the pool
            self.storage.copy_slots(g, src, dst, slots)

    # ------------------------------------------------------------------ admission
    def _plan(self, tokens: Sequence[int], max_new: int | None, reuse_limit: int | None) -> _Admission:
        """
        Read-only.  The demand on a pool is the most pages it has to give at any moment of the
        admission and the request's later growth, counted as pages leaving `available()`:
        an idle page that is taken over leaves it just as a blank page that is taken does.
        """
        B = self.page_tokens
        total = len(tokens)
        reuse = self.index.lookup(tokens, reuse_limit) if self.index is not None else Reuse([])
        reserve = total - reuse.num_tokens if max_new is None else min(total - reuse.num_tokens, max_new)
        whole_request = -(-total // B)
        copy_from = None
        demand = []
        for p, pool in enumerate(self.pools):
            if self.window_of_pool[p]:
                demand.append(-(-(reuse.num_tokens + reserve) // B))     # later portions find pages the window has passed
            elif self.index is None or p != self.shared:
                demand.append(whole_request)
            else:
                refs = pool.refs
                if reuse.run:                              # a page in use cannot be evicted under the copy: prefer one
                    copy_from = min(reuse.starting_with_run, key=lambda c: (refs[c.page] == 0, c.page))
                woken = sum(1 for c in reuse.pages if refs[c.page] == 0)   # idle pages that come back into use
                taken = whole_request - len(reuse.pages)    # blank pages over the request's life, the copy's target among them
                last = reuse.pages[-1] if reuse.pages else None
                if last is not None and not last.is_full(B) and refs[last.page] > 0:
                    taken += 1                             # its holder writes there too: the request will write into a copy
                if copy_from is not None and refs[copy_from.page] == 0:
                    taken = max(taken, 2)                  # source and target exist side by side while the copy is made
                demand.append(woken + taken)
        return _Admission(reuse, copy_from, reserve, tuple(demand), total - reuse.num_tokens)

    def admission_cost(self, tokens: Sequence[int], max_new: int | None = None,
                       reuse_limit: int | None = None) -> AdmissionCost:
        """What admitting these tokens would take from the pools and how many tokens it would run.  Read-only."""
        plan = self._plan(tokens, max_new, reuse_limit)
        return AdmissionCost(plan.demand, plan.prefill_tokens)

    def admit(self, seq_id: int, tokens: Sequence[int], max_new: int | None = None,
              reuse_limit: int | None = None) -> bool:
        """
        Starts a request: takes over the recorded start of its tokens, copies the run a further
        page begins with, takes a state slot and reserves slots for the next `max_new` tokens
        (None: all the rest).  Returns False, changing nothing, if the pools cannot hold the whole
        request right now.  `reuse_limit`: at most this many leading tokens are taken from the
        cache (a caller that wants the model's output at a prompt position must have it run).
        """
        assert len(tokens) > 0, "a request needs at least one token"
        assert seq_id not in self.seqs, "the request is admitted already"
        plan = self._plan(tokens, max_new, reuse_limit)
        if not self.fits(plan.demand) or (self.layout.state_bytes and not self._free_slots):
            return False
        seq = SeqState(tables=[[] for _ in self.pools])
        if plan.reuse.pages or plan.copy_from is not None:
            pool, table = self.pools[self.shared], seq.tables[self.shared]
            for cached in plan.reuse.pages:                # first all of them: a held page cannot be evicted below
                pool.hold(cached.page)
                table.append(cached.page)
            if plan.copy_from is not None:
                source = plan.copy_from.page
                pool.hold(source)
                target = pool.take()
                self._copy(self.shared, source, target, plan.reuse.run)
                pool.let_go(source)                        # the copy is ordered on the stream before any reuse of the page
                table.append(target)
                self.counters.partial_copies += 1
        seq.committed = plan.reuse.num_tokens
        seq.tokens = list(tokens[:seq.committed])
        if self.layout.state_bytes:
            seq.state_slot = self._free_slots.pop()
            self.storage.clear_state(seq.state_slot)
        self.seqs[seq_id] = seq
        self._reserve(seq, tokens[seq.committed:seq.committed + plan.reserve])
        return True

    # ------------------------------------------------------------------ reservation
    def _shares_last_page(self, seq: SeqState, p: int) -> bool:
        """The next token would land in a partly filled page that somebody else holds as well."""
        table = seq.tables[p]
        return bool(seq.reserved % self.page_tokens and table and table[-1] >= 0 and self.pools[p].refs[table[-1]] > 1)

    def _growth(self, seq: SeqState, n: int) -> tuple[int, ...]:
        """Pages each pool has to give for `n` more tokens of this request."""
        pages_then = -(-(seq.reserved + n) // self.page_tokens)
        return tuple(max(0, pages_then - len(seq.tables[p]) + self._shares_last_page(seq, p)) for p in range(len(self.pools)))

    def pages_needed_to_extend(self, seq_id: int, n: int) -> tuple[int, ...]:
        return self._growth(self.seqs[seq_id], n)

    def can_extend(self, seq_id: int, n: int) -> bool:
        return self.fits(self._growth(self.seqs[seq_id], n))

    def pages_for_one_more_each(self, seq_ids: Sequence) -> list[int]:
        """Per pool, the pages that one more token for each of these requests would take: one pass, for large batches."""
        B = self.page_tokens
        total = [0] * len(self.pools)
        for seq_id in seq_ids:
            seq = self.seqs[seq_id]
            fill = len(seq.tokens) % B
            for p, table in enumerate(seq.tables):
                if fill == 0:
                    total[p] += 1                          # the token opens a page
                elif table[-1] >= 0 and self.pools[p].refs[table[-1]] > 1:
                    total[p] += 1                          # the token goes into a copy of the shared page
        return total

    def extend(self, seq_id: int, tokens: Sequence[int], checked: bool = False) -> None:
        """
        Reserves slots for the step's tokens of a running request; commit() closes the step.
        `checked`: the caller has made sure the pages are there (pages_for_one_more_each + fits).
        """
        assert len(tokens) > 0, "a step feeds at least one token"
        seq = self.seqs[seq_id]
        assert len(seq.tokens) == seq.committed, "the previous step was not committed"
        if not checked and not self.fits(self._growth(seq, len(tokens))):
            raise CacheFull("not enough free pages: check can_extend() first")
        self._reserve(seq, tokens)

    def _reserve(self, seq: SeqState, tokens: Sequence[int]) -> None:
        B = self.page_tokens
        fill = seq.reserved % B
        pages_then = -(-(seq.reserved + len(tokens)) // B)
        for p, pool in enumerate(self.pools):
            table = seq.tables[p]
            if self._shares_last_page(seq, p):             # copy on write
                mine = pool.take()
                self._copy(p, table[-1], mine, fill)
                pool.let_go(table[-1])
                table[-1] = mine
                self.counters.cow_copies += 1
            elif fill and table and table[-1] >= 0:
                cached = pool.cached(table[-1])
                assert cached is None or fill >= len(cached.tokens), "a slot on record would be overwritten"
            table.extend(pool.take() for _ in range(pages_then - len(table)))
        seq.tokens.extend(tokens)

    # ------------------------------------------------------------------ commit / release / fork
    def commit(self, seq_id: int, num_accepted: int) -> None:
        """
        Closes a step: keeps the first `num_accepted` slots reserved since the last commit, drops the
        rest, puts pages that became full on record, and gives back pages a window has passed.
        """
        seq = self.seqs[seq_id]
        fed = seq.reserved - seq.committed
        assert 0 <= num_accepted <= fed, "more slots accepted than reserved"
        assert not self.layout.state_bytes or num_accepted == fed, "a model with per-request state cannot take back tokens it has run"
        assert PENDING_TOKEN not in seq.tokens[seq.committed:seq.committed + num_accepted], \
            "a token still pending would be committed: amend it first"
        B = self.page_tokens
        first_new_page = seq.committed // B
        seq.committed += num_accepted
        del seq.tokens[seq.committed:]
        pages_kept = -(-seq.committed // B)
        for p, pool in enumerate(self.pools):
            table = seq.tables[p]
            for page in table[pages_kept:]:                # pages only rejected tokens reached
                if page >= 0:
                    pool.let_go(page)
            del table[pages_kept:]
            window = self.window_of_pool[p]
            if window:
                # the next query sits at position `committed` and sees keys from committed - window + 1 on
                passed = min(max(0, seq.committed - window + 1) // B, len(table))
                for i in range(passed):
                    if table[i] >= 0:
                        pool.let_go(table[i])
                        table[i] = -1
                        self.counters.window_releases += 1
        if self.index is not None:
            for i in range(first_new_page, seq.committed // B):
                self._record(seq, i)

    def _record(self, seq: SeqState, i: int) -> None:
        """
        Puts page `i` of the request on record with the committed tokens it holds.  If the index
        knows a page with the same tokens at the same place, the request reads that one from now
        on and gives its own back: two requests computed the same page, one copy is kept.
        """
        B = self.page_tokens
        pool, table = self.pools[self.shared], seq.tables[self.shared]
        mine = table[i]
        held = tuple(seq.tokens[i * B:min((i + 1) * B, seq.committed)])
        entry = self.index.by_page.get(mine)
        if entry is None:
            under = self.index.by_page[table[i - 1]] if i else self.index.root
            kept = self.index.file(under, mine, held)
            if kept.page == mine:
                self.counters.publishes += 1
        elif len(entry.tokens) < len(held):
            kept = self.index.lengthen(entry, held)
        else:
            return
        if kept.page != mine:
            pool.hold(kept.page)
            table[i] = kept.page
            pool.let_go(mine)
            self.counters.dedupes += 1

    def amend_last(self, seq_id: int, token: int) -> None:
        """Fills in the one reserved token that was extended as PENDING_TOKEN, before its commit."""
        seq = self.seqs[seq_id]
        assert seq.reserved == seq.committed + 1 and seq.tokens[-1] == PENDING_TOKEN, "no pending token to amend"
        seq.tokens[-1] = token

    def release(self, seq_id: int, drop_reserved: bool = False) -> None:
        """
        Ends a request (finished or preempted).  With prefix reuse everything it committed stays on
        record, the partly filled last page too, until the pool needs the pages.  `drop_reserved`:
        slots reserved for a step that will not be committed go with it (a request that ended
        while its next step was already launched).
        """
        seq = self.seqs[seq_id]
        assert drop_reserved or seq.reserved == seq.committed, "release between steps: commit first"
        del seq.tokens[seq.committed:]
        if self.index is not None and seq.committed % self.page_tokens:
            self._record(seq, seq.committed // self.page_tokens)
        del self.seqs[seq_id]
        for pool, table in zip(self.pools, seq.tables):
            # from the end: a page is let go of before the page it continues from, so of an idle chain the end
            # is always the stalest part and goes first
            for page in reversed(table):
                if page >= 0:
                    pool.let_go(page)
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
        for pool, table in zip(self.pools, src.tables):
            for page in table:
                if page >= 0:
                    pool.hold(page)
        self.seqs[new_id] = SeqState(tables=[list(t) for t in src.tables], tokens=list(src.tokens),
                                     committed=src.committed, state_slot=slot)
