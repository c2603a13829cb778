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
            for g, table in enumerate(seq.tables):
                page = table[pos // B]
                assert page >= 0, "a token is written into a page that was given back"
                self.slots[g][page][pos % B] = seq.tokens[pos]
            if seq.state_slot >= 0:
                self.state[seq.state_slot].append(seq.tokens[pos])


def layout_of(page_tokens=4, windows=(0,), state_bytes=0) -> CacheLayout:
    groups = tuple(GroupLayout((i,), 2, 16, w) for i, w in enumerate(windows))
    offsets = tuple(0 if state_bytes and i == 0 else -1 for i in range(len(windows)))
    return CacheLayout(page_tokens, groups, offsets, state_bytes, tuple(state_bytes if o == 0 else 0 for o in offsets))


def check_invariants(manager: CacheManager, storage: FakeStorage) -> None:
    B = manager.page_tokens
    for g, pool in enumerate(manager.pools):
        holders = Counter(p for s in manager.seqs.values() for p in s.tables[g] if p >= 0)
        for page in range(pool.num_pages):
            assert pool.refs[page] == holders.get(page, 0), f"group {g} page {page}: ref {pool.refs[page]} vs holders"
        free = list(pool.free) + list(pool.free_cached)
        assert len(free) == len(set(free)), "a page is free twice"
        assert set(free) == {p for p in range(pool.num_pages) if pool.refs[p] == 0}, "a page is lost or held while free"
        for page in pool.free_cached:
            assert g == 0 and page in manager.tree.nodes
        for page in pool.free:
            assert g != 0 or page not in manager.tree.nodes
    # the tree: chained, partial pages are leaves, contents are what the tree says, held pages have held parents
    refs0 = manager.pools[0].refs if manager.pools else []
    for page, node in manager.tree.nodes.items():
        assert node.page == page and 0 < len(node.tokens) <= B
        assert node.parent.children[node.tokens] is node
        if len(node.tokens) < B:
            assert not node.children, "a partly filled page has children"
        assert tuple(storage.slots[0][page][:len(node.tokens)]) == node.tokens, "cached page does not hold its tokens"
        if refs0[page] > 0 and node.parent.page >= 0:
            assert refs0[node.parent.page] > 0, "a held page's parent is free"
    used_slots = [s.state_slot for s in manager.seqs.values() if s.state_slot >= 0]
    assert len(used_slots) == len(set(used_slots)), "two requests share a state slot"
    assert not set(used_slots) & set(manager._free_slots), "a state slot is free while in use"
    for seq in manager.seqs.values():
        for g, group in enumerate(manager.layout.groups):
            table = seq.tables[g]
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
        if manager.caching:
            for i in range(seq.committed // B):
                assert seq.tables[0][i] in manager.tree.nodes, "a full committed page is not in the tree"
        if seq.state_slot >= 0:
            assert storage.state[seq.state_slot] == seq.tokens[:seq.committed], "state does not follow the tokens"
