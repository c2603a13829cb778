"""
The step function: one batch of (request, its next tokens) through the model, from the cache.

A step may hold portions of prompts beside single decoded tokens, cut anywhere.  It runs only the
tokens it is given, as one flat batch, against the keys and values earlier steps left in the pages,
and returns float32 logits at the wanted places.  The caller reserves the tokens' slots in the cache
manager before the step (admit / extend) and commits them after it; the step reads the block
tables, which may have changed since the last step, afresh each time.

tinyserve-llm packs a step the same way (engine/model_runner.py:43-89: flat ids, positions, slots,
block tables, sample rows) and returns sampled tokens; here the step returns logits and sampling is
a separate call, so that a replay can ask for any row.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import torch

from tinyserve_llm_b200.cache.manager import CacheManager
from tinyserve_llm_b200.cache.storage import DeviceCacheStorage, EntryBinding
from tinyserve_llm_b200.config.spec import RunEntry
from tinyserve_llm_b200.parts.model import DecoderModel


@dataclass
class StepEntry:
    """One request's share of a step: the tokens it feeds and the places among them whose logits are wanted."""

    seq_id: int
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)    # indices into `tokens`


@dataclass
class HostView:
    """The step's index data as Python lists, for parts whose code runs on the host (toy and test mixers)."""

    seq_ids: list[int]
    cu_q: list[int]              # [S + 1] offsets of each request's tokens in the flat batch
    start: list[int]             # [S] position of each request's first token in this step
    ctx_lens: list[int]          # [S] keys per request after this step's writes
    state_slots: list[int]       # [S] state slot per request (-1: none)


class StepContext:
    """What the parts see of a step."""

    def __init__(self, runner: "StepRunner", num_tokens: int, num_seqs: int, host: HostView) -> None:
        self._runner = runner
        self.num_tokens = num_tokens
        self.num_seqs = num_seqs
        self.host = host
        self.token_ids: torch.Tensor = None       # int32 [T]
        self.positions: torch.Tensor = None       # int32 [T]
        self.seq_of_token: torch.Tensor = None    # int32 [T]; -1 marks a padding row
        self.cu_q: torch.Tensor = None            # int32 [S + 1]
        self.ctx_lens: torch.Tensor = None        # int32 [S]
        self.state_slots: torch.Tensor = None     # int32 [S]
        self.rows: torch.Tensor = None            # int32 [R] flat rows whose logits are wanted
        self.tables: list[torch.Tensor] = []      # per group int32 [S, width]
        self.max_q_len = max((b - a for a, b in zip(host.cu_q, host.cu_q[1:])), default=0)
        self.max_ctx_len = max(host.ctx_lens, default=0)

    def binding(self, entry: RunEntry) -> EntryBinding | None:
        base = self._runner.bindings[entry.cache_entry]
        if base is None:
            return None
        table = self.tables[base.group] if base.group >= 0 else None
        return EntryBinding(base.k_pool, base.v_pool, base.page_stride, base.entry_offset, base.page_tokens,
                            base.num_pages, table, table.shape[1] if table is not None else 0,
                            entry.writes_cache, base.group, base.state, self.state_slots)


def _pad4(n: int) -> int:
    return (n + 3) & ~3


class StepRunner:
    def __init__(self, model: DecoderModel, manager: CacheManager, storage: DeviceCacheStorage) -> None:
        self.model = model
        self.manager = manager
        self.storage = storage
        self.device = model.rt.device
        self.bindings = [storage.entry_binding(e) for e in range(model.spec.num_cache_entries)]
        self._staging: torch.Tensor | None = None       # pinned int32 buffer for the step's index data
        self._staged = torch.cuda.Event()
        self._staged.record()

    # ------------------------------------------------------------------ packing
    def _validate(self, entries: Sequence[StepEntry]) -> None:
        if not entries:
            raise ValueError("a step needs at least one entry")
        vocab, max_pos = self.model.spec.vocab_size, self.model.spec.max_positions
        seen = set()
        for e in entries:
            if e.seq_id in seen:
                raise ValueError(f"request {e.seq_id!r} appears twice in one step")
            seen.add(e.seq_id)
            if e.seq_id not in self.manager.seqs:
                raise KeyError(f"request {e.seq_id!r} has no reservation in the cache manager")
            n = len(e.tokens)
            if n == 0:
                raise ValueError(f"request {e.seq_id!r} feeds no token")
            state = self.manager.seqs[e.seq_id]
            if state.reserved - state.committed != n:
                raise ValueError(f"request {e.seq_id!r} feeds {n} tokens but reserved "
                                 f"{state.reserved - state.committed}")
            if state.committed + n > max_pos:
                raise ValueError(f"request {e.seq_id!r} would reach position {state.committed + n - 1}; "
                                 f"the model's position table has {max_pos}")
            lo, hi = min(e.tokens), max(e.tokens)
            if lo < 0 or hi >= vocab:
                raise ValueError(f"request {e.seq_id!r}: token id {lo if lo < 0 else hi} outside the vocabulary of {vocab}")
            for w in e.want:
                if not 0 <= w < n:
                    raise ValueError(f"request {e.seq_id!r}: wanted place {w} outside its {n} tokens")

    def _pack(self, entries: Sequence[StepEntry]) -> StepContext:
        mgr = self.manager
        ids: list[int] = []
        positions: list[int] = []
        seq_of_token: list[int] = []
        cu_q, start, ctx_lens, rows, slots, seq_ids = [0], [], [], [], [], []
        for s, e in enumerate(entries):
            state = mgr.seqs[e.seq_id]
            n = len(e.tokens)
            first = state.committed
            ids.extend(e.tokens)
            positions.extend(range(first, first + n))
            seq_of_token.extend([s] * n)
            rows.extend(cu_q[-1] + w for w in e.want)
            cu_q.append(cu_q[-1] + n)
            start.append(first)
            ctx_lens.append(first + n)
            slots.append(state.state_slot)
            seq_ids.append(e.seq_id)
        T, S, R = len(ids), len(entries), len(rows)
        groups = len(mgr.pools)
        widths = [max(1, max(len(mgr.seqs[e.seq_id].tables[g]) for e in entries)) for g in range(groups)]
        sections = [ids, positions, seq_of_token, cu_q, ctx_lens, rows, slots]
        for g in range(groups):
            flat: list[int] = []
            for e in entries:
                t = mgr.seqs[e.seq_id].tables[g]
                flat.extend(t)
                flat.extend([-1] * (widths[g] - len(t)))
            sections.append(flat)
        offsets, total = [], 0
        for sec in sections:
            offsets.append(total)
            total += _pad4(max(len(sec), 1))
        if self._staging is None or self._staging.numel() < total:
            self._staging = torch.empty(max(total, 4096), dtype=torch.int32).pin_memory()
        else:
            self._staged.synchronize()                  # the previous step's copy has read the buffer
        host = self._staging
        for off, sec in zip(offsets, sections):
            if sec:
                host[off:off + len(sec)] = torch.tensor(sec, dtype=torch.int32)
        dev = host[:total].to(self.device, non_blocking=True)
        self._staged.record()

        ctx = StepContext(self, T, S, HostView(seq_ids, cu_q, start, ctx_lens, slots))
        view = lambda i, n: dev[offsets[i]:offsets[i] + n]  # noqa: E731
        ctx.token_ids, ctx.positions, ctx.seq_of_token = view(0, T), view(1, T), view(2, T)
        ctx.cu_q, ctx.ctx_lens, ctx.rows, ctx.state_slots = view(3, S + 1), view(4, S), view(5, R), view(6, S)
        ctx.tables = [view(7 + g, S * widths[g]).view(S, widths[g]) for g in range(groups)]
        return ctx

    # ------------------------------------------------------------------ the step
    @torch.inference_mode()
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """float32 [wanted places, vocab] on the device, in the order of the entries and of their `want`."""
        self._validate(entries)
        ctx = self._pack(entries)
        x, residual = self.model.forward(ctx)
        if ctx.rows.numel() == 0:
            return torch.empty((0, self.model.spec.vocab_size), dtype=torch.float32, device=self.device)
        return self.model.logits(x, residual, ctx.rows)
