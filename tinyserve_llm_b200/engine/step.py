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
    feed: int = -1      # >= 0: the entry's one token is element `feed` of the step's `device_tokens`; `tokens` is a placeholder


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
        self.prefill_seqs: torch.Tensor = None    # int32 [P] requests that feed more than one token (prompt portions)
        self.tables: list[torch.Tensor] = []      # per pool of the cache manager int32 [S, width]
        lens = [b - a for a, b in zip(host.cu_q, host.cu_q[1:])]
        self.max_q_len = max(lens, default=0)     # which attention kernels a step needs is decided on the host
        self.min_q_len = min(lens, default=0)
        self.max_ctx_len = max(host.ctx_lens, default=0)   # an upper bound; a replayed step sets its shape's bound
        # the split-key decode kernels size their grid and scratch by the longest request that feeds one token
        self.max_decode_ctx_len = max((c for c, n in zip(host.ctx_lens, lens) if n == 1), default=0)
        self.scratch: dict = {}                   # per-step scratch buffers parts share (keyed by purpose and size)

    def binding(self, entry: RunEntry) -> EntryBinding | None:
        base = self._runner.bindings[entry.cache_entry]
        if base is None:
            return None
        table = self.tables[self._runner.manager.pool_of_group[base.group]] if base.group >= 0 else None
        return EntryBinding(base.k_pool, base.v_pool, base.page_stride, base.entry_offset, base.page_tokens,
                            base.num_pages, table, table.shape[1] if table is not None else 0,
                            entry.writes_cache, base.group, base.state, self.state_slots)


GRAPH_MAX_TOKENS = 512      # the largest step with a prompt portion that is replayed from a graph (see StepRunner)


def _pad4(n: int) -> int:
    return (n + 3) & ~3


def _power_of_two(n: int) -> int:
    b = 1
    while b < n:
        b *= 2
    return b


@dataclass(frozen=True)
class StepShape:
    """
    The sizes a step replayed from a CUDA graph is padded to: what its kernels' grids and its
    buffers are sized by.  Real tokens come first, then padding rows (seq_of_token = -1); real
    requests first, then padding requests that feed nothing; the list of prompt portions is
    padded with -1.
    """

    tokens: int                 # rows of the flat batch
    seqs: int                   # requests; also the number of logits rows the graph computes
    portions: int               # entries of the list of requests that feed more than one token (0: none)
    max_q: int                  # bound on the longest portion (1: every request feeds one token)
    decodes: bool               # some request feeds exactly one token: the split-key kernels run
    widths: tuple[int, ...]     # block-table width per pool of the cache manager


class _StepGraph:
    """A captured step of one shape: static index buffer in, rows of the runner's static logits buffer out."""

    def __init__(self, graph: torch.cuda.CUDAGraph, index_buffer: torch.Tensor, logits: torch.Tensor,
                 shape: StepShape, launches: int) -> None:
        self.graph = graph
        self.index_buffer = index_buffer
        self.logits = logits
        self.shape = shape
        self.widths = list(shape.widths)
        self.launches = launches       # kernels of the engine's own library inside the graph


class StepRunner:
    """
    `cuda_graphs`: steps are replayed from CUDA graphs where every part of the model is graph safe.
    A graph is captured per `StepShape`, the step's sizes rounded up to buckets:

    * steps in which every request feeds one token (decoding): batch size in powers of two, block
      tables as wide as the step's longest request needs (1, 2, 3, 4, 6, 8, 12, ... pages: the
      attention's grid covers what the tables can hold, and tables for the longest context the
      engine allows made 64 requests of 512 tokens cost 3.4 ms a step instead of 1.26);
    * steps with prompt portions of up to `graph_max_tokens` tokens in all: tokens in multiples of
      64, requests, portions and the longest portion in powers of two.  Launched kernel by kernel
      such a step costs about 2 ms of host time whatever its size, more than its device time below
      a few hundred tokens (Llama 3.2 1B sizes); from about 512 tokens on the device takes longer
      than the host and a graph gains nothing.  A capture costs several steps' time, so a shape is
      captured when it is met the third time: a replay of conversations whose prompts all differ
      in length met two thirds of its shapes once or twice only.

    Larger steps, steps that want more logits rows than they have requests, and models with a part
    that is not graph safe run eagerly.  The logits a replayed step returns live in one static
    buffer that all graphs write ([largest batch bucket, vocab] float32, allocated at the first
    capture) and are overwritten by the next replayed step: consume them (sample, copy) before
    stepping again.  At most `max_graphs` graphs are kept; the least recently used one goes first.
    `table_pages` (per layer group) stands in for the pools' page counts where the widest block
    table is worked out: a runner on a small throwaway pool can then capture the graphs the real
    pool will need.
    """

    def __init__(self, model: DecoderModel, manager: CacheManager, storage: DeviceCacheStorage, *,
                 cuda_graphs: bool = True, max_decode_batch: int = 256, max_model_len: int | None = None,
                 max_graphs: int = 64, table_pages: Sequence[int] | None = None, graph_max_tokens: int = GRAPH_MAX_TOKENS,
                 sightings_before_capture: int = 3) -> None:
        self.model = model
        self.manager = manager
        self.storage = storage
        self.device = model.rt.device
        self.bindings = [storage.entry_binding(e) for e in range(model.spec.num_cache_entries)]
        self._staging: torch.Tensor | None = None       # pinned int32 buffer for the step's index data
        self._staged = torch.cuda.Event()
        self._staged.record()
        self.cuda_graphs = bool(cuda_graphs) and model.graph_safe
        self.max_decode_batch = max_decode_batch
        self.graph_max_tokens = graph_max_tokens
        self.sightings_before_capture = sightings_before_capture
        longest = min(max_model_len or model.spec.max_positions, model.spec.max_positions)
        pool_pages = list(table_pages) if table_pages is not None else [pool.num_pages for pool in manager.pools]
        self._graph_widths = [max(1, min(pages, -(-longest // manager.page_tokens))) for pages in pool_pages]
        self._graph_logits: torch.Tensor | None = None   # [largest batch bucket, vocab] float32, shared by all graphs
        self._graphs: dict[StepShape, _StepGraph] = {}   # least recently used first
        self._met: dict[StepShape, int] = {}             # shapes with portions seen so far and not captured yet
        self.max_graphs = max_graphs
        self._graph_pool = None                          # the graphs' intermediates share one memory pool
        self.last_graph: _StepGraph | None = None
        self.steps = 0                                   # steps run so far, of which ...
        self.graph_replays = 0                           # ... from a graph (the step that captured one included) ...
        self.graph_captures = 0                          # ... and how many graphs were captured; the rest was launched kernel by kernel
        self.eager_tokens = 0                            # tokens of the steps launched kernel by kernel

    # ------------------------------------------------------------------ packing
    def _validate(self, entries: Sequence[StepEntry], device_tokens: torch.Tensor | None = None) -> None:
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
            if e.feed >= 0:
                if n != 1 or device_tokens is None or e.feed >= device_tokens.shape[0]:
                    raise ValueError(f"request {e.seq_id!r}: a token fed on the device is one token, element "
                                     f"{e.feed} of a `device_tokens` tensor that holds it")
                lo = hi = 0
            else:
                lo, hi = min(e.tokens), max(e.tokens)
            if lo < 0 or hi >= vocab:
                raise ValueError(f"request {e.seq_id!r}: token id {lo if lo < 0 else hi} outside the vocabulary of {vocab}")
            for w in e.want:
                if not 0 <= w < n:
                    raise ValueError(f"request {e.seq_id!r}: wanted place {w} outside its {n} tokens")

    def _index_data(self, entries: Sequence[StepEntry], shape: StepShape | None) -> tuple[list[int], list[int], dict]:
        """
        The step's index data as one list of int32 words in sections (each padded to 16 bytes):
        token ids, positions, request of each token, offsets of the requests' tokens, lengths after
        this step, wanted rows, state slots, one block table per pool of the cache manager, and the requests
        that feed more than one token.  With `shape`, every section is padded to the shape's size.
        Returns (words, offset of each section, sizes).
        """
        seqs = self.manager.seqs
        states = [seqs[e.seq_id] for e in entries]
        n = len(entries)
        groups = len(self.manager.pools)
        if all(len(e.tokens) == 1 for e in entries):            # decoding: no loop over tokens
            first = [st.committed for st in states]
            ids = [e.tokens[0] if e.feed < 0 else -(e.feed + 2) for e in entries]
            positions = first
            seq_of_token = list(range(n))
            cu_q = list(range(n + 1))
            ctx_lens = [f + 1 for f in first]
            rows = [i for i, e in enumerate(entries) if len(e.want)]
            portions: list[int] = []
        else:
            ids, positions, seq_of_token, cu_q, ctx_lens, rows, portions = [], [], [], [0], [], [], []
            for s, (e, st) in enumerate(zip(entries, states)):
                k = len(e.tokens)
                begin = st.committed
                ids.extend(e.tokens if e.feed < 0 else (-(e.feed + 2),))
                positions.extend(range(begin, begin + k))
                seq_of_token.extend([s] * k)
                at = cu_q[-1]
                rows.extend(at + w for w in e.want)
                cu_q.append(at + k)
                ctx_lens.append(begin + k)
                if k > 1:
                    portions.append(s)
        slots = [st.state_slot for st in states]
        T, R, P = len(ids), len(rows), len(portions)
        if shape is None:
            widths = [max(1, max(len(st.tables[g]) for st in states)) for g in range(groups)]
            S = n
        else:
            widths, S = list(shape.widths), shape.seqs
            if T > shape.tokens or n > S or R > S or P > shape.portions:
                raise ValueError("the step does not fit the shape it was bucketed into")
            pad = shape.tokens - T
            ids = ids + [0] * pad
            positions = positions + [0] * pad
            seq_of_token = seq_of_token + [-1] * pad
            cu_q = cu_q + [T] * (S - n)                          # padding requests feed nothing
            ctx_lens = ctx_lens + [0] * (S - n)
            slots = slots + [-1] * (S - n)
            rows = rows + [0] * (S - R)
            portions = portions + [-1] * (shape.portions - P)
        sections = [ids, positions, seq_of_token, cu_q, ctx_lens, rows, slots]
        for g in range(groups):
            flat: list[int] = []
            width = widths[g]
            for e, st in zip(entries, states):
                t = st.tables[g]
                if len(t) > width:
                    raise ValueError(f"request {e.seq_id!r} holds {len(t)} pages; the step was built for {width}")
                flat.extend(t)
                if len(t) < width:
                    flat.extend([-1] * (width - len(t)))
            if S > n:
                flat.extend([-1] * (width * (S - n)))
            sections.append(flat)
        sections.append(portions)
        offsets, words = [], []
        for sec in sections:
            offsets.append(len(words))
            words.extend(sec)
            pad = _pad4(max(len(sec), 1)) - len(sec)
            if pad:
                words.extend([0] * pad)
        sizes = dict(tokens=len(ids), seqs=S, rows=len(rows), portions=len(portions), widths=widths, real_tokens=T,
                     real_seqs=n, real_rows=R, real_portions=P, cu_q=cu_q, ctx_lens=ctx_lens, slots=slots)
        return words, offsets, sizes

    def _upload(self, words: list[int], into: torch.Tensor | None) -> torch.Tensor:
        """One conversion, one copy into the pinned buffer, one copy to the device (into a graph's static buffer, if given)."""
        total = len(words)
        if self._staging is None or self._staging.numel() < total:
            self._staging = torch.empty(max(total, 4096), dtype=torch.int32).pin_memory()
        else:
            self._staged.synchronize()                  # the previous step's copy has read the buffer
        host = self._staging
        host[:total] = torch.tensor(words, dtype=torch.int32)
        if into is None:
            dev = host[:total].to(self.device, non_blocking=True)
        else:
            dev = into
            dev[:total].copy_(host[:total], non_blocking=True)
        self._staged.record()
        return dev

    def _pack(self, entries: Sequence[StepEntry], shape: StepShape | None = None,
              into: torch.Tensor | None = None) -> StepContext:
        """The step's context: its index data on the device and what the host knows of it."""
        words, offsets, sizes = self._index_data(entries, shape)
        dev = self._upload(words, into)
        n = sizes["real_seqs"]
        cu_q, ctx_lens = sizes["cu_q"], sizes["ctx_lens"]
        host = HostView([e.seq_id for e in entries], cu_q[:n + 1], [c - (b - a) for a, b, c in zip(cu_q, cu_q[1:], ctx_lens[:n])],
                        ctx_lens[:n], sizes["slots"][:n])
        ctx = StepContext(self, sizes["tokens"], sizes["seqs"], host)
        ctx.index_words = len(words)
        if shape is not None:                     # a graph is replayed for any step its shape can hold
            bound = max(w * self.manager.page_tokens for w in shape.widths) if shape.widths else 0
            ctx.max_q_len, ctx.min_q_len = shape.max_q, (1 if shape.decodes else shape.max_q)
            ctx.max_ctx_len = ctx.max_decode_ctx_len = bound
        T, S, R, P = sizes["tokens"], sizes["seqs"], sizes["rows"], sizes["portions"]
        widths = sizes["widths"]
        view = lambda i, k: dev[offsets[i]:offsets[i] + k]  # noqa: E731
        ctx.token_ids, ctx.positions, ctx.seq_of_token = view(0, T), view(1, T), view(2, T)
        ctx.cu_q, ctx.ctx_lens, ctx.rows, ctx.state_slots = view(3, S + 1), view(4, S), view(5, R), view(6, S)
        groups = len(widths)
        ctx.tables = [view(7 + g, S * widths[g]).view(S, widths[g]) for g in range(groups)]
        ctx.prefill_seqs = view(7 + groups, P)
        return ctx

    # ------------------------------------------------------------------ the step
    @torch.inference_mode()
    def step(self, entries: Sequence[StepEntry], device_tokens: torch.Tensor | None = None) -> torch.Tensor:
        """
        float32 [wanted places, vocab] on the device, in the order of the entries and of their `want`.

        `device_tokens` (int32, on the device) serves entries with `feed` >= 0: their token is read
        from it on the device, so a decode step can be launched before the host has seen the
        previous step's samples.
        """
        self._validate(entries, device_tokens)
        self.model.rt.ops.check_device_errors()      # a bounded wait that ran out in an earlier step (host-visible word)
        self.steps += 1
        shape = self.graph_shape(entries) if self.cuda_graphs else None
        if shape is not None:
            captured = self._graphs.pop(shape, None)
            if captured is not None:
                self._graphs[shape] = captured               # most recently used last
                return self._replay(captured, entries, device_tokens)
            met = self._met.get(shape, 0) + 1
            if shape.portions == 0 or met >= self.sightings_before_capture:
                self._met.pop(shape, None)
                return self._replay(self._capture(entries, shape, device_tokens), entries, None, launched=True)
            if len(self._met) > 4 * self.max_graphs:
                self._met.clear()
            self._met[shape] = met
        ctx = self._pack(entries)
        self.eager_tokens += ctx.num_tokens
        if device_tokens is not None:
            self.model.rt.ops.feed_tokens(ctx.token_ids, device_tokens)
        x, residual = self.model.forward(ctx)
        if ctx.rows.numel() == 0:
            return torch.empty((0, self.model.spec.vocab_size), dtype=torch.float32, device=self.device)
        return self.model.logits(x, residual, ctx.rows)

    # ------------------------------------------------------------------ steps from CUDA graphs
    @staticmethod
    def bucket(n: int) -> int:
        return _power_of_two(n)

    @staticmethod
    def width_bucket(pages: int) -> int:
        """Block-table widths of graphs: 1, 2, 3, 4, 6, 8, 12, 16, 24, ... (at most half again what is needed)."""
        b = 1
        while b < pages:
            if b >= 2 and b + b // 2 >= pages:
                return b + b // 2
            b *= 2
        return b

    def graph_shape(self, entries: Sequence[StepEntry]) -> StepShape | None:
        """The shape this step would be replayed in; None where it runs eagerly."""
        n = len(entries)
        if n > self.max_decode_batch:
            return None
        tokens = rows = portions = longest = 0
        decodes = False
        for e in entries:
            k = len(e.tokens)
            tokens += k
            rows += len(e.want)
            if k > 1:
                portions += 1
                longest = max(longest, k)
            else:
                decodes = True
        seqs = _power_of_two(n)
        if rows > seqs:
            return None
        states = self.manager.seqs
        widths = tuple(min(limit, self.width_bucket(max(len(states[e.seq_id].tables[g]) for e in entries)))
                       for g, limit in enumerate(self._graph_widths))
        if portions == 0:
            return StepShape(seqs, seqs, 0, 1, True, widths)
        if tokens > self.graph_max_tokens:
            return None
        padded = -(-tokens // 64) * 64
        return StepShape(padded, seqs, _power_of_two(portions), min(padded, max(64, _power_of_two(longest))), decodes, widths)

    def _replay(self, captured: _StepGraph, entries: Sequence[StepEntry], device_tokens: torch.Tensor | None,
                launched: bool = False) -> torch.Tensor:
        if not launched:
            words, _, _ = self._index_data(entries, captured.shape)
            self._upload(words, captured.index_buffer)
            if device_tokens is not None:
                self.model.rt.ops.feed_tokens(captured.index_buffer[:captured.shape.tokens], device_tokens)
            captured.graph.replay()
            self.model.rt.ops.launches += captured.launches
        self.graph_replays += 1
        self.last_graph = captured
        return captured.logits[:sum(len(e.want) for e in entries)]

    def _capture(self, entries: Sequence[StepEntry], shape: StepShape,
                 device_tokens: torch.Tensor | None = None) -> _StepGraph:
        words, _, _ = self._index_data(entries, shape)
        index_buffer = torch.empty(len(words), dtype=torch.int32, device=self.device)
        ctx = self._pack(entries, shape, into=index_buffer)
        if device_tokens is not None:
            self.model.rt.ops.feed_tokens(ctx.token_ids, device_tokens)
        if self._graph_logits is None:
            self._graph_logits = torch.empty((self.bucket(self.max_decode_batch), self.model.spec.vocab_size),
                                             dtype=torch.float32, device=self.device)
        out = self._graph_logits[:shape.seqs]
        # once eagerly: libraries create their handles and workspaces outside the capture, and this run IS
        # the step (its keys and values are written, its logits are in the static buffer); the capture
        # that follows records the same launches without running them
        x, residual = self.model.forward(ctx)
        self.model.logits(x, residual, ctx.rows, out=out)
        torch.cuda.synchronize(self.device)
        # Scratch buffers the parts put into the context during the eager run came from the ordinary allocator and
        # go back to it when this context is dropped: the capture must not record their addresses (a replay would
        # write into memory that by then belongs to someone else, or to nobody).  It allocates its own, from the
        # graphs' pool.
        del x, residual
        ctx.scratch.clear()
        graph = torch.cuda.CUDAGraph()
        ops = self.model.rt.ops
        before = ops.launches
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        with torch.cuda.graph(graph, pool=self._graph_pool):
            x, residual = self.model.forward(ctx)
            logits = self.model.logits(x, residual, ctx.rows, out=out)
        launches = ops.launches - before
        captured = _StepGraph(graph, index_buffer, logits, shape, launches)
        self.graph_captures += 1
        while len(self._graphs) >= self.max_graphs:
            self._graphs.pop(next(iter(self._graphs)))
        self._graphs[shape] = captured
        return captured
