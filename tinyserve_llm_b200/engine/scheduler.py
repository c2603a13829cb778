"""
The scheduler: admits requests, cuts prompts into portions under a token budget, decodes, finishes
and frees.

Policy follows tinyserve-llm (scheduler/scheduler.py:12-267): waiting requests are ranked by
score = cache hit + wait_weight * seconds waited; every running sequence that is decoding gets its
token first; admissions fill what is left of `max_num_batched_tokens`, under the sequence cap and a
watermark of free pages; a candidate that does not fit is skipped until it has waited
`max_skip_wait` seconds, after which admission stops so that freed pages go to it; a group of n
samples forks after the step that ran its prompt's last token.

New here, prompts run in portions: a running sequence whose tokens are not all in the cache takes
min(what is left, `prefill_chunk`, the budget left) tokens per step and samples only in the step
that runs its last token, so `max_num_batched_tokens` may be smaller than a prompt.

When pages run out.  A decode that needs a page preempts the lowest-scoring running sequence not
yet scheduled in this step (or itself, if none is left): the victim's pages are released (they stay
cached for reuse), it returns to the waiting queue with its outputs and arrival time, and is later
run again from its whole token list.  A prompt portion that finds no page waits for a later step.
If a step would otherwise be empty while sequences are running, the lowest-scoring one is preempted
and the step is built again; a step that is empty with nothing running raises in the engine.

Running ahead (new here).  While a step is still on the device, `schedule_ahead` may decide the
step after it: a sequence that samples in the step under way feeds the token it is about to
sample, which the engine passes from step to step on the device, and a sequence still in its
prompt feeds its next portion.  It does so only where the decision does not depend on the samples:
nothing waits (or nothing waiting could be admitted: the sequence cap is full, or the last
admission pass found room for none and nothing has made room since), everything running is in the
step, no group forks, and the pages the next step takes are free.  A sequence that reaches
`max_tokens` in the step under way is left out.  The one thing unknown is an end-of-sequence token:
a sequence that samples one finishes as usual, its pages are released, and its share of the step
launched ahead is thrown away.

The policy (what is ranked how, who gives way, what an admission must leave free) is
tinyserve-llm's; how a step is put together here is this engine's own: a draft that is filled by
decodes, prompt portions and admissions in turn, room for decodes made by one count over the
whole batch, and admission conditions kept as the seats, pages and state slots that are left.
"""

from __future__ import annotations

import itertools
import math
from dataclasses import dataclass, replace
from typing import NamedTuple

from tinyserve_llm_b200.cache.manager import PENDING_TOKEN, AdmissionCost, CacheManager
from tinyserve_llm_b200.engine.sequence import SamplingParams, Sequence, SequenceStatus


@dataclass(frozen=True)
class SchedulerConfig:
    max_model_len: int = 4096
    max_num_seqs: int = 512
    max_num_batched_tokens: int = 16384
    eos_token_id: int = -1
    wait_weight: float = 0.1
    hit_mode: str = "absolute"            # "absolute": cached tokens / max_model_len; "ratio": / request length
    max_skip_wait: float = 5.0
    watermark: float = 0.01
    step_mode: str = "mixed"              # "mixed" or "prefill_first"
    prefill_chunk: int = 2048             # most prompt tokens of one sequence in one step; 0: no limit

    def __post_init__(self) -> None:
        if self.hit_mode not in ("absolute", "ratio"):
            raise ValueError(f"hit_mode must be 'absolute' or 'ratio', got {self.hit_mode!r}")
        if self.step_mode not in ("mixed", "prefill_first"):
            raise ValueError(f"step_mode must be 'mixed' or 'prefill_first', got {self.step_mode!r}")
        if self.max_model_len < 2 or self.max_num_seqs < 1 or self.prefill_chunk < 0:
            raise ValueError("max_model_len >= 2, max_num_seqs >= 1 and prefill_chunk >= 0 are required")
        if self.max_num_batched_tokens < self.max_num_seqs:
            raise ValueError("max_num_batched_tokens must leave one token for each of max_num_seqs decodes")
        if not 0.0 <= self.watermark < 1.0:
            raise ValueError("watermark is a fraction of the pool in [0, 1)")


@dataclass
class SchedulerStats:
    """Running totals since start; the two queue sizes are current values."""

    admissions: int = 0
    readmissions: int = 0
    preemptions: int = 0
    cached_tokens: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    stalled_portions: int = 0     # prompt portions that waited a step for pages
    num_waiting: int = 0
    num_running: int = 0


class ScheduledSeq(NamedTuple):
    seq: Sequence
    token_ids: list[int]          # positions start at the sequence's committed length
    num_samples: int = 1          # 0: a prompt portion that does not reach the last token; n on a group's first sampling step


class RequestOutput(NamedTuple):
    request_id: int
    sequences: list[Sequence]


class _Draft:
    """A step being put together: what is in it, and what is left of the token budget."""

    def __init__(self, tokens_left: int) -> None:
        self.entries: list[ScheduledSeq] = []
        self.tokens_left = tokens_left

    def add(self, seq: Sequence, tokens: list[int], num_samples: int) -> None:
        self.entries.append(ScheduledSeq(seq, tokens, num_samples))
        self.tokens_left -= len(tokens)


class Candidate(NamedTuple):
    """A waiting sequence as an admission pass sees it."""

    seq: Sequence
    tokens: list[int]             # prompt and, after a preemption, the outputs so far
    cost: AdmissionCost
    hit: float
    priority: float


class Scheduler:
    def __init__(self, config: SchedulerConfig, cache: CacheManager) -> None:
        self.config = config
        self.cache = cache
        self.waiting: list[Sequence] = []
        self.running: list[Sequence] = []
        self.groups: dict[int, list[Sequence]] = {}
        self.watermark_pages = math.ceil(config.watermark * cache.num_pages)
        self._seq_ids = itertools.count()
        self._request_ids = itertools.count()
        self.counters = SchedulerStats()
        # True from an admission pass that found room for none of the waiting requests until something that
        # could make room happens (a request arrives, ends or is preempted, a window gives pages back):
        # pages are only taken meanwhile, so the pass would come out the same
        self._nothing_admissible = False
        self._window_releases_seen = 0

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    def stats(self) -> SchedulerStats:
        return replace(self.counters, num_waiting=len(self.waiting), num_running=len(self.running))

    # ------------------------------------------------------------------ intake
    def _never_fits(self, length: int, params: SamplingParams) -> str | None:
        """Why a request of `length` tokens at its longest could not run even with the engine to itself."""
        if length > self.config.max_model_len:
            return f"prompt + max_tokens = {length} exceeds max_model_len = {self.config.max_model_len}"
        # at its longest: its own pages, one copied page per further sample, what admissions must leave free, and the
        # page that holds a partly matching cached page while its slots are copied
        pages = -(-length // self.cache.page_tokens) + (params.n - 1) + self.watermark_pages + 1
        if pages > self.cache.num_pages:
            return f"needs up to {pages} pages; the cache has {self.cache.num_pages}"
        if params.n > self.config.max_num_seqs:
            return f"n = {params.n} samples exceed max_num_seqs = {self.config.max_num_seqs}"
        return None

    def add_request(self, prompt_token_ids: list[int], params: SamplingParams, arrival_time: float) -> int:
        """Queues a request and returns its id; rejects one that could never run."""
        if not prompt_token_ids:
            raise ValueError("a request needs at least one prompt token")
        if params.max_tokens < 1 or params.n < 1:
            raise ValueError("max_tokens and n must be at least 1")
        if params.temperature < 0:
            raise ValueError("temperature must not be negative")
        problem = self._never_fits(len(prompt_token_ids) + params.max_tokens, params)
        if problem is not None:
            raise ValueError(problem)
        request_id = next(self._request_ids)
        seq = Sequence(next(self._seq_ids), request_id, tuple(prompt_token_ids), params, arrival_time)
        self.groups[request_id] = [seq]
        self.waiting.append(seq)
        self._nothing_admissible = False
        return request_id

    # ------------------------------------------------------------------ priority
    def priority(self, seq: Sequence, now: float, hit: float | None = None) -> float:
        """
        Cache hit plus weighted wait (scheduler/scheduler.py:89-117 of tinyserve-llm): a waiting
        sequence is ranked by the hit it would have now, a running one keeps the hit it was admitted
        with, and both keep ageing from their arrival.
        """
        return (seq.admission_hit if hit is None else hit) + self.config.wait_weight * (now - seq.arrival_time)

    def _candidate(self, seq: Sequence, now: float) -> Candidate:
        tokens = seq.all_token_ids
        cost = self.cache.admission_cost(tokens)
        scale = self.config.max_model_len if self.config.hit_mode == "absolute" else len(tokens)
        hit = (len(tokens) - cost.prefill_tokens) / scale
        return Candidate(seq, tokens, cost, hit, self.priority(seq, now, hit))

    def waiting_by_rank(self, now: float) -> list[Candidate]:
        """The waiting sequences, best first; earlier arrival breaks a tie."""
        candidates = [self._candidate(seq, now) for seq in self.waiting]
        order = sorted(range(len(candidates)), key=lambda i: (-candidates[i].priority, i))
        return [candidates[i] for i in order]

    def _lowest(self, seqs: list[Sequence], now: float) -> Sequence:
        return min(seqs, key=lambda s: self.priority(s, now))

    # ------------------------------------------------------------------ what a sequence does next
    def _left_to_run(self, seq: Sequence) -> int:
        return seq.num_tokens - self.cache.committed_tokens(seq.seq_id)

    def _decoding(self, seq: Sequence) -> bool:
        return bool(seq.output_token_ids) and self._left_to_run(seq) == 1

    def _portion(self, left_to_run: int, tokens_left: int) -> int:
        n = min(left_to_run, tokens_left)
        return min(n, self.config.prefill_chunk) if self.config.prefill_chunk else n

    @staticmethod
    def _samples_after(seq: Sequence, reaches_end: bool) -> int:
        """How many tokens are drawn after a step: none inside a prompt, n where a group's prompt ends, else one."""
        if not reaches_end:
            return 0
        return seq.params.n if (seq.params.n > 1 and not seq.output_token_ids) else 1

    # ------------------------------------------------------------------ putting a step together
    def schedule(self, now: float) -> list[ScheduledSeq]:
        while True:
            draft = self._draft(now)
            if draft.entries or not self.running:
                return draft.entries
            self._preempt(self._lowest(self.running, now))      # everything running waits for pages: one gives way

    def _draft(self, now: float) -> _Draft:
        draft = _Draft(self.config.max_num_batched_tokens)
        if self.config.step_mode == "prefill_first":
            self._add_portions(draft, now)
            self._add_admissions(draft, now)
            if not draft.entries:
                self._add_decodes(draft, now)
        else:
            self._add_decodes(draft, now)
            self._add_portions(draft, now)
            self._add_admissions(draft, now)
        return draft

    def _add_decodes(self, draft: _Draft, now: float) -> None:
        """
        Every decoding sequence feeds its last token.  If the pages their next tokens need are not all
        there (counted in one pass over the batch), the lowest-ranked running sequence gives way, decoding
        or still in its prompt, until they are; decodes may use what admissions have to leave free.
        """
        decoding = [s for s in self.running if self._decoding(s)]
        while decoding and not self.cache.fits(self.cache.pages_for_one_more_each([s.seq_id for s in decoding])):
            victim = self._lowest(self.running, now)
            self._preempt(victim)
            if victim in decoding:
                decoding.remove(victim)
        decoding.sort(key=lambda s: -self.priority(s, now))
        for seq in decoding:
            token = seq.output_token_ids[-1]
            self.cache.extend(seq.seq_id, [token], checked=True)
            draft.add(seq, [token], 1)
        self.counters.decode_tokens += len(decoding)

    def _add_portions(self, draft: _Draft, now: float) -> None:
        """Sequences still in their prompt (or recomputing after a preemption) feed their next portion, best first."""
        in_prompt = [s for s in self.running if not self._decoding(s)
                     and self.cache.reserved_tokens(s.seq_id) == self.cache.committed_tokens(s.seq_id)]
        in_prompt.sort(key=lambda s: -self.priority(s, now))
        for seq in in_prompt:
            if draft.tokens_left <= 0:
                break
            left = self._left_to_run(seq)
            n = self._portion(left, draft.tokens_left)
            if not self.cache.can_extend(seq.seq_id, n):
                self.counters.stalled_portions += 1              # waits for pages; a later step takes it up
                continue
            begin = seq.num_tokens - left
            tokens = seq.all_token_ids[begin:begin + n]
            self.cache.extend(seq.seq_id, tokens)
            self.counters.prefill_tokens += n
            draft.add(seq, tokens, self._samples_after(seq, n == left))

    def _preempt(self, seq: Sequence) -> None:
        """The sequence gives its pages back (they stay cached) and waits again, with its outputs and its arrival time."""
        self.running.remove(seq)
        self.cache.release(seq.seq_id)
        seq.status = SequenceStatus.WAITING
        seq.num_preemptions += 1
        self.counters.preemptions += 1
        self.waiting.append(seq)
        self._nothing_admissible = False

    def _add_admissions(self, draft: _Draft, now: float) -> None:
        """
        Waiting sequences in rank order, while the draft has tokens left.  One is admitted if a seat, the
        pages and a state slot are there for it and for the further samples its group will fork into, with
        the watermark left free; a misfit is passed over while young, and ends the pass once it has waited
        `max_skip_wait`, so that what comes free goes to it (scheduler/scheduler.py:160-204 of tinyserve-llm).
        """
        considered = draft.tokens_left > 0 and bool(self.waiting)
        seats = self.config.max_num_seqs - len(self.running)
        forks_owed = 0                       # further samples of groups admitted in this pass: each takes a page and a slot later
        admitted: list[Sequence] = []
        for candidate in self.waiting_by_rank(now):
            if draft.tokens_left <= 0:
                break
            if admitted:                     # an admission may have evicted what this one's hit counted on
                candidate = self._candidate(candidate.seq, now)
            seq, tokens, cost = candidate.seq, candidate.tokens, candidate.cost
            branches = seq.params.n - 1 if (seq.params.n > 1 and not seq.output_token_ids) else 0
            room = (seats >= 1 + branches
                    and self.cache.fits(cost.pages_needed, forks_owed + branches + self.watermark_pages)
                    and self.cache.free_state_slots() >= 1 + forks_owed + branches)
            if not room:
                if now - seq.arrival_time >= self.config.max_skip_wait:
                    break
                continue
            n = self._portion(cost.prefill_tokens, draft.tokens_left)
            started = self.cache.admit(seq.seq_id, tokens, n)
            assert started, "the room was checked against a fresh cost"
            cached = self.cache.committed_tokens(seq.seq_id)
            fed = tokens[cached:cached + n]
            if seq.num_preemptions:
                self.counters.readmissions += 1
            else:
                self.counters.admissions += 1
            self.counters.cached_tokens += cached
            self.counters.prefill_tokens += len(fed)
            seats -= 1 + branches
            forks_owed += branches
            seq.status = SequenceStatus.RUNNING
            seq.admission_hit = candidate.hit
            self.running.append(seq)
            admitted.append(seq)
            draft.add(seq, fed, self._samples_after(seq, cached + len(fed) == len(tokens)))
        if admitted:
            gone = {s.seq_id for s in admitted}
            self.waiting = [s for s in self.waiting if s.seq_id not in gone]
        self._nothing_admissible = considered and not admitted
        self._window_releases_seen = self.cache.counters.window_releases

    # ------------------------------------------------------------------ the step after the one under way
    def schedule_ahead(self, under_way: list[ScheduledSeq]) -> list[ScheduledSeq] | None:
        """
        The step that follows `under_way`, whose samples are not known yet; None where that step
        depends on them (then nothing is changed).  Otherwise `under_way` is committed here (its
        tokens are known, and whatever reads their keys is launched after it), each sequence that
        samples in it reserves one slot with PENDING_TOKEN as its token, each sequence still in
        its prompt its next portion, and `postprocess` is told so.
        """
        alive = [e for e in under_way if e.seq.status is SequenceStatus.RUNNING]
        if any(e.num_samples > 1 for e in alive):
            return None                          # a group forks once its samples are known
        if {e.seq.seq_id for e in alive} != {s.seq_id for s in self.running}:
            return None                          # somebody running sat the step out: a full pass decides what is next
        # the step under way gives a sampling sequence output number len(outputs) + 1
        samplers = [e.seq for e in alive if e.num_samples and len(e.seq.output_token_ids) + 1 < e.seq.params.max_tokens]
        in_prompt = [e.seq for e in alive if not e.num_samples]
        ending = len(alive) - len(samplers) - len(in_prompt)
        if not samplers and not in_prompt:
            return None
        if in_prompt and self.config.step_mode == "prefill_first":
            return None                          # such a step holds the prompts alone; the sequences that sample sit it out
        # Requests that wait rule the step out unless none of them could be admitted into it anyway: nobody
        # reaches max_tokens in the step under way, and either the sequence cap is full or the last admission
        # pass found room for none of them and nothing has made room since.  A request that ends on an
        # end-of-sequence token then hands its place on one step later than it would have.
        if self.waiting:
            if ending:
                return None
            stuck = self._nothing_admissible and self._window_releases_seen == self.cache.counters.window_releases
            if not stuck and len(self.running) < self.config.max_num_seqs:
                return None
        # the pages of the whole step, or nothing: who gives way is decided when the tokens are known
        tokens_left = self.config.max_num_batched_tokens - len(samplers)
        portions: list[tuple[Sequence, int, int]] = []
        need = self.cache.pages_for_one_more_each([s.seq_id for s in samplers])
        for seq in sorted(in_prompt, key=lambda s: -self.priority(s, 0.0)):
            left = seq.num_tokens - self.cache.reserved_tokens(seq.seq_id)     # what is reserved is under way
            n = self._portion(left, tokens_left)
            if n <= 0:
                return None
            need = [a + b for a, b in zip(need, self.cache.pages_needed_to_extend(seq.seq_id, n))]
            portions.append((seq, left, n))
            tokens_left -= n
        if not self.cache.fits(need):
            return None
        for e in alive:
            self.cache.commit(e.seq.seq_id, len(e.token_ids))
        ahead = _Draft(self.config.max_num_batched_tokens)
        unknown = [PENDING_TOKEN]
        for seq in samplers:
            self.cache.extend(seq.seq_id, unknown, checked=True)
            ahead.add(seq, unknown, 1)
        self.counters.decode_tokens += len(samplers)
        for seq, left, n in portions:
            begin = seq.num_tokens - left
            tokens = seq.all_token_ids[begin:begin + n]
            self.cache.extend(seq.seq_id, tokens, checked=True)
            self.counters.prefill_tokens += n
            ahead.add(seq, tokens, self._samples_after(seq, n == left))
        return ahead.entries

    # ------------------------------------------------------------------ after the model ran
    def _branch(self, parent: Sequence, index: int) -> Sequence:
        """A further sample of a group: a sequence of its own that shares every page of the prompt."""
        child = Sequence(next(self._seq_ids), parent.request_id, parent.prompt_token_ids, parent.params,
                         parent.arrival_time, status=SequenceStatus.RUNNING, sample_index=index,
                         admission_hit=parent.admission_hit)
        self.cache.fork(parent.seq_id, child.seq_id)
        self.running.append(child)
        self.groups[parent.request_id].append(child)
        return child

    def _deliver(self, seq: Sequence, token: int, now: float, reserved_ahead: bool) -> bool:
        """Books one sampled token; True if the sequence ends with it (an end-of-sequence token is kept)."""
        seq.output_token_ids.append(token)
        if seq.first_token_time is None:
            seq.first_token_time = now
        if token == self.config.eos_token_id and not seq.params.ignore_eos:
            seq.finish_reason = "eos"
        elif len(seq.output_token_ids) >= seq.params.max_tokens:
            seq.finish_reason = "length"
        else:
            return False
        self.cache.release(seq.seq_id, drop_reserved=reserved_ahead)
        seq.status = SequenceStatus.FINISHED
        seq.finish_time = now
        return True

    def postprocess(self, scheduled: list[ScheduledSeq], sampled: list[list[int]], now: float,
                    ahead: list[ScheduledSeq] | None = None) -> list[RequestOutput]:
        """
        Closes the step, lets groups fork where their prompt ended, books the tokens and frees what
        finished.  `ahead` is what `schedule_ahead(scheduled)` returned: the step is committed
        already, and the sequences that feed an unknown token in `ahead` get it filled in.  Samples
        of a sequence that finished while this step was launched ahead are dropped.
        """
        in_ahead = {e.seq.seq_id for e in ahead} if ahead is not None else set()
        fed_unknown = {e.seq.seq_id for e in ahead if e.token_ids[0] == PENDING_TOKEN} if ahead is not None else set()
        ended: list[Sequence] = []
        for (seq, token_ids, num_samples), tokens in zip(scheduled, sampled, strict=True):
            assert len(tokens) == num_samples
            if seq.status is SequenceStatus.FINISHED:
                continue
            if ahead is None:
                self.cache.commit(seq.seq_id, len(token_ids))
            elif seq.seq_id in fed_unknown:
                self.cache.amend_last(seq.seq_id, tokens[0])
            samples = [seq] + [self._branch(seq, i) for i in range(1, num_samples)] if num_samples else []
            for sample, token in zip(samples, tokens):
                if self._deliver(sample, token, now, sample.seq_id in in_ahead):
                    ended.append(sample)
        if ended:
            gone = {s.seq_id for s in ended}
            self.running = [s for s in self.running if s.seq_id not in gone]
            self._nothing_admissible = False
        outputs = []
        for request_id in dict.fromkeys(s.request_id for s in ended):
            group = self.groups[request_id]
            if len(group) == group[0].params.n and all(s.status is SequenceStatus.FINISHED for s in group):
                outputs.append(RequestOutput(request_id, self.groups.pop(request_id)))
        return outputs
