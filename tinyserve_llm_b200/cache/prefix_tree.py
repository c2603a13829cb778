"""
Prefix index over published cache pages: a tree with one node per page, and under every node an
index of its children by their leading tokens, so that a new prompt reuses cached keys and values
token by token.

Behaviour follows tinyserve-llm's page tree (kvcache/page_tree.py:43-128, kvcache/trie.py:28-69):
a walk matches whole pages by their exact token tuple, then asks the last node's trie for the
longest run of leading tokens some child shares; the last token of a prompt is never matched, so
an admitted request always feeds at least one token; only full pages have children; only leaves
are evicted.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Iterable, Sequence


def _common_prefix(a: tuple, b: tuple) -> int:
    """Length of the longest common prefix of two tuples; the comparisons run at C speed on slices."""
    n = min(len(a), len(b))
    if a[:n] == b[:n]:
        return n
    lo, hi = 0, n                              # a[:lo] == b[:lo] and a[:hi] != b[:hi]
    while hi - lo > 1:
        mid = (lo + hi) // 2
        if a[lo:mid] == b[lo:mid]:
            lo = mid
        else:
            hi = mid
    return lo


class TokenTrie:
    """
    Children of one page, indexed by their leading tokens.  It answers what a trie over the
    children's tokens answers (kvcache/trie.py:28-69 of the reference), but keeps no node per
    token: a child is filed under its first token with its token tuple, and the longest shared run
    is found by comparing tuples when it is asked for.  Publishing a page then costs one dictionary
    entry instead of one object per token.
    """

    __slots__ = ("by_first",)

    def __init__(self) -> None:
        self.by_first: dict[int, dict[object, tuple[int, ...]]] = {}

    def add(self, page: "PageNode", tokens: Sequence[int]) -> None:
        """Index `page` under `tokens`; adding a longer run for the same page replaces the shorter one."""
        tokens = tuple(tokens)
        self.by_first.setdefault(tokens[0], {})[page] = tokens

    def discard(self, page: "PageNode", tokens: Sequence[int]) -> None:
        """Remove `page`, which was added under `tokens` (or under a run `tokens` extends)."""
        bucket = self.by_first[tokens[0]]
        del bucket[page]
        if not bucket:
            del self.by_first[tokens[0]]

    def longest_run(self, tokens: Sequence[int]) -> tuple[int, set["PageNode"]]:
        """(number of leading tokens matched, the children that share that run; read-only)."""
        tokens = tuple(tokens)
        bucket = self.by_first.get(tokens[0]) if tokens else None
        if not bucket:
            return 0, set()
        best, sharing = 0, set()
        for page, recorded in bucket.items():
            depth = _common_prefix(tokens, recorded)
            if depth > best:
                best, sharing = depth, {page}
            elif depth == best:
                sharing.add(page)
        return best, sharing


@dataclass(eq=False)
class PageNode:
    page: int                                   # page id in the pool; -1 for the root
    tokens: tuple[int, ...]                     # tokens whose keys/values the page holds; only grows
    parent: "PageNode | None"
    children: dict[tuple[int, ...], "PageNode"] = field(default_factory=dict)
    trie: TokenTrie = field(default_factory=TokenTrie)
    stamp: int = 0                              # release time, for least-recently-used eviction


@dataclass
class PrefixMatch:
    pages: list[PageNode]                       # attached whole (each over all its recorded tokens)
    partial_len: int = 0                        # further tokens found inside some other page
    partial_sources: frozenset[PageNode] = frozenset()

    @property
    def num_tokens(self) -> int:
        return sum(len(p.tokens) for p in self.pages) + self.partial_len


class PrefixTree:
    def __init__(self, page_tokens: int) -> None:
        self.page_tokens = page_tokens
        self.root = PageNode(page=-1, tokens=(), parent=None)
        self.nodes: dict[int, PageNode] = {}

    def match(self, tokens: Sequence[int]) -> PrefixMatch:
        """The longest cached prefix of tokens[:-1]."""
        limit = len(tokens) - 1
        node, pos = self.root, 0
        found: list[PageNode] = []
        while pos < limit:
            chunk = tuple(tokens[pos:min(pos + self.page_tokens, limit)])
            child = node.children.get(chunk)
            if child is not None:
                found.append(child)
                pos += len(chunk)
                node = child
                continue
            depth, sharing = node.trie.longest_run(chunk)
            if depth == 0:
                break
            whole = next((p for p in sharing if len(p.tokens) == depth), None)
            if whole is not None:                # a partly filled page matched over all it holds
                found.append(whole)
                break
            return PrefixMatch(found, depth, frozenset(sharing))
        return PrefixMatch(found)

    def publish(self, parent: PageNode, page: int, tokens: Iterable[int]) -> PageNode:
        """Add `page` under `parent`; returns the node holding `tokens` (an older one if it exists)."""
        tokens = tuple(tokens)
        assert 0 < len(tokens) <= self.page_tokens
        assert parent is self.root or len(parent.tokens) == self.page_tokens, "only full pages have children"
        assert page not in self.nodes, "the page is in the tree already; grow it instead"
        older = parent.children.get(tokens)
        if older is not None:
            return older
        node = PageNode(page=page, tokens=tokens, parent=parent)
        parent.children[tokens] = node
        parent.trie.add(node, tokens)
        self.nodes[page] = node
        return node

    def grow(self, node: PageNode, tokens: Iterable[int]) -> PageNode:
        """Extend a partly filled page in place; returns a sibling instead if one holds `tokens` already."""
        tokens = tuple(tokens)
        old = node.tokens
        assert len(old) < len(tokens) <= self.page_tokens and tokens[:len(old)] == old
        parent = node.parent
        assert parent is not None
        sibling = parent.children.get(tokens)
        if sibling is not None:
            return sibling
        del parent.children[old]
        node.tokens = tokens
        parent.children[tokens] = node
        parent.trie.add(node, tokens)
        return node

    def evict(self, node: PageNode) -> int:
        """Remove a leaf; returns its page id."""
        assert not node.children, "only leaves are evicted"
        parent = node.parent
        assert parent is not None
        removed = parent.children.pop(node.tokens)
        assert removed is node
        parent.trie.discard(node, node.tokens)
        del self.nodes[node.page]
        return node.page
