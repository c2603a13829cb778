"""A storage fake whose page slots hold token ids, and the cache manager's full contract as one check."""

from __future__ import annotations

from collections import Counter

from tinyserve_llm_b200.cache import CacheLayout, CacheManager, GroupLayout


class FakeStorage:
    """Slots hold the token whose key/value would be there, so a misplaced read or copy shows."""

    def __init__(self, layout: CacheLayout, num_pages: list[int], num_state_slots: int = 0) -> None:
        self.page_tokens = layout.page_tokens
        self.slots = [[[None] * layout.page_tokens for _ in range(n)] for n in num_pages]
        self.state = [None] * num_state_slots
        self.copies = []

    def copy_slots(self, group, src, dst, n):
        self.copies.append((group, src, dst, n))
        self.slots[group][dst][:n] = self.slots[group][src][:n]

    def copy_state(self, src, dst):
        self.state[dst] = list(self.state[src])

    def clear_state(self, slot):
        self.state[slot] = []

    def run_step(self, manager: CacheManager, seq_id) -> None:
        """What the model's step does: writes every reserved, uncommitted token into its slot."""
        seq = manager.seqs[seq_id]
        B = self.page_tokens
        for pos in range(seq.committed, seq.reserved):
            for g, pool in enumerate(manager.pool_of_group):          # every layer group writes its own tensors
                page = seq.tables[pool][pos // B]
                assert page >= 0, "a token is written into a page that was given back"
                self.slots[g][page][pos % B] = seq.tokens[pos]
            if seq.state_slot >= 0:
                self.state[seq.state_slot].append(seq.tokens[pos])


def layout_of(page_tokens=4, windows=(0,), state_bytes=0) -> CacheLayout:
    groups = tuple(GroupLayout((i,), 2, 16, w) for i, w in enumerate(windows))
    offsets = tuple(0 if state_bytes and i == 0 else -1 for i in range(len(windows)))
    return CacheLayout(page_tokens, groups, offsets, state_bytes, tuple(state_bytes if o == 0 else 0 for o in offsets))


def check_invariants(manager: CacheManager, storage: FakeStorage) -> None:
    """
    No page lost, held twice or freed twice; the record of cached pages says what the pages hold;
    every token a request may still read is where its table says; windows and state slots as promised.
    """
    B = manager.page_tokens
    index = manager.index
    for p, pool in enumerate(manager.pools):
        holders = Counter(page for s in manager.seqs.values() for page in s.tables[p] if page >= 0)
        for page in range(pool.num_pages):
            assert pool.refs[page] == holders.get(page, 0), f"pool {p} page {page}: ref {pool.refs[page]} vs holders"
        free = pool.blank_pages() + pool.idle_pages()
        assert len(free) == len(set(free)), "a page is free twice"
        assert set(free) == {page for page in range(pool.num_pages) if pool.refs[page] == 0}, "a page is lost or held while free"
        assert pool.available() == len(free)
        for page in pool.idle_pages():
            assert pool.index is not None and page in pool.index.by_page, "an idle page is not on record"
        for page in pool.blank_pages():
            assert pool.index is None or page not in pool.index.by_page, "a blank page is on record"
    if index is not None:
        refs = manager.pools[manager.shared].refs
        for page, entry in index.by_page.items():
            assert entry.page == page and 0 < len(entry.tokens) <= B
            assert entry in entry.before.after
            if len(entry.tokens) < B:
                assert not entry.after, "a partly filled page is continued"
            keys = [e.tokens for e in entry.after]
            assert keys == sorted(keys) and len(set(keys)) == len(keys), "the pages after a page are out of order"
            for g in manager.groups_of_pool[manager.shared]:
                assert tuple(storage.slots[g][page][:len(entry.tokens)]) == entry.tokens, "cached page does not hold its tokens"
            if refs[page] > 0 and entry.before.page >= 0:
                assert refs[entry.before.page] > 0, "a held page continues from a free one"
        # every idle page can be reached by evicting from the ends: an idle page has no held page behind it
        for page in manager.pools[manager.shared].idle_pages():
            assert all(refs[e.page] == 0 for e in index.by_page[page].after)
    used_slots = [s.state_slot for s in manager.seqs.values() if s.state_slot >= 0]
    assert len(used_slots) == len(set(used_slots)), "two requests share a state slot"
    assert not set(used_slots) & set(manager._free_slots), "a state slot is free while in use"
    for seq in manager.seqs.values():
        for g, group in enumerate(manager.layout.groups):
            table = seq.tables[manager.pool_of_group[g]]
            assert len(table) == -(-seq.reserved // B)
            first_needed = max(0, seq.committed - group.window + 1) if group.window else 0
            for pos in range(seq.committed):
                page = table[pos // B]
                if pos >= first_needed:
                    assert page >= 0, "a page inside the window was given back"
                    assert storage.slots[g][page][pos % B] == seq.tokens[pos], \
                        f"group {g}: slot of position {pos} holds {storage.slots[g][page][pos % B]}, not {seq.tokens[pos]}"
            if group.window:
                for i, page in enumerate(table):
                    if (i + 1) * B <= first_needed:
                        assert page == -1, "a page behind the window is still held"
        if index is not None:
            for i in range(seq.committed // B):
                assert seq.tables[manager.shared][i] in index.by_page, "a full committed page is not on record"
        if seq.state_slot >= 0:
            assert storage.state[seq.state_slot] == seq.tokens[:seq.committed], "state does not follow the tokens"
