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

Running ahead (new here).  While a decode step is still on the device, `schedule_ahead` may decide
the step after it: every running sequence feeds the token it is about to sample, which the engine
passes from step to step on the device.  It does so only where the decision does not depend on
those tokens: nothing waits (or nothing waiting could be admitted: the sequence cap is full, or the last
admission pass found room for none and nothing has made room since), everything running is in the step
and samples one token, and the pages for one more token each are free.  A sequence that reaches `max_tokens` in the step under way is
left out.  The one thing unknown is an end-of-sequence token: a sequence that samples one finishes
as usual, its pages are released, and its share of the step launched ahead is thrown away.
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

    # ------------------------------------------------------------------ intake
    def add_request(self, prompt_token_ids: list[int], params: SamplingParams, arrival_time: float) -> int:
        """Queues a request and returns its id; rejects one that could never run."""
        if not prompt_token_ids:
            raise ValueError("a request needs at least one prompt token")
        if params.max_tokens < 1 or params.n < 1:
            raise ValueError("max_tokens and n must be at least 1")
        if params.temperature < 0:
            raise ValueError("temperature must not be negative")
        longest = len(prompt_token_ids) + params.max_tokens
        if longest > self.config.max_model_len:
            raise ValueError(f"prompt + max_tokens = {longest} exceeds max_model_len = {self.config.max_model_len}")
        # one sequence at full length, a copied page per fork, the watermark, and one page that
        # holds a partly matching cached page while its slots are copied
        worst = -(-longest // self.cache.page_tokens) + (params.n - 1) + self.watermark_pages + 1
        if worst > self.cache.num_pages:
            raise ValueError(f"needs up to {worst} pages; the cache has {self.cache.num_pages}")
        if params.n > self.config.max_num_seqs:
            raise ValueError(f"n = {params.n} samples exceed max_num_seqs = {self.config.max_num_seqs}")
        request_id = next(self._request_ids)
        seq = Sequence(next(self._seq_ids), request_id, tuple(prompt_token_ids), params, arrival_time)
        self.groups[request_id] = [seq]
        self.waiting.append(seq)
        self._nothing_admissible = False
        return request_id

    # ------------------------------------------------------------------ ranking
    def _hit(self, num_tokens: int, cost: AdmissionCost) -> float:
        cached = num_tokens - cost.prefill_tokens
        return cached / (self.config.max_model_len if self.config.hit_mode == "absolute" else num_tokens)

    def _score(self, hit: float, seq: Sequence, now: float) -> float:
        return hit + self.config.wait_weight * (now - seq.arrival_time)

    def _ranked_waiting(self, now: float) -> list[tuple[Sequence, AdmissionCost, float]]:
        ranked = []
        for order, seq in enumerate(self.waiting):
            tokens = seq.all_token_ids
            cost = self.cache.admission_cost(tokens)
            hit = self._hit(len(tokens), cost)
            ranked.append((-self._score(hit, seq, now), order, seq, cost, hit))
        ranked.sort(key=lambda r: (r[0], r[1]))
        return [(seq, cost, hit) for _, _, seq, cost, hit in ranked]

    def _portion(self, remaining: int, budget: int) -> int:
        n = min(remaining, budget)
        if self.config.prefill_chunk:
            n = min(n, self.config.prefill_chunk)
        return n

    # ------------------------------------------------------------------ building a step
    def schedule(self, now: float) -> list[ScheduledSeq]:
        while True:
            batch = self._build(now)
            if batch or not self.running:
                return batch
            # everything running is stalled for pages: free the lowest-scoring one and try again
            victim = min(self.running, key=lambda s: self._score(s.admission_hit, s, now))
            self.running.remove(victim)
            self._preempt(victim)

    def _build(self, now: float) -> list[ScheduledSeq]:
        budget = self.config.max_num_batched_tokens
        if self.config.step_mode == "prefill_first":
            first = self._continue_prefills(now, budget)
            budget -= sum(len(s.token_ids) for s in first)
            first += self._admit(now, budget)
            return first or self._schedule_decodes(now)
        decodes = self._schedule_decodes(now)
        budget -= len(decodes)
        portions = self._continue_prefills(now, budget)
        budget -= sum(len(s.token_ids) for s in portions)
        return decodes + portions + self._admit(now, budget)

    def _remaining(self, seq: Sequence) -> int:
        return seq.num_tokens - self.cache.committed_tokens(seq.seq_id)

    def _is_decoding(self, seq: Sequence) -> bool:
        return bool(seq.output_token_ids) and self._remaining(seq) == 1

    def _schedule_decodes(self, now: float) -> list[ScheduledSeq]:
        decoding = [s for s in self.running if self._is_decoding(s)]
        others = [s for s in self.running if not self._is_decoding(s)]
        queue = sorted(decoding, key=lambda s: self._score(s.admission_hit, s, now))    # lowest score first
        scheduled: list[ScheduledSeq] = []
        kept: list[Sequence] = []
        while queue:
            seq = queue.pop()                                    # highest score left
            while not self.cache.can_extend(seq.seq_id, 1) and queue:
                self._preempt(queue.pop(0))
            if not self.cache.can_extend(seq.seq_id, 1):
                # nothing decoding ranks lower; a sequence still in its prompt may give way instead
                victim = min(others, key=lambda s: self._score(s.admission_hit, s, now), default=None)
                if victim is not None and self._score(victim.admission_hit, victim, now) < \
                        self._score(seq.admission_hit, seq, now):
                    others.remove(victim)
                    self._preempt(victim)
                if not self.cache.can_extend(seq.seq_id, 1):
                    self._preempt(seq)
                    break
            token = seq.output_token_ids[-1]
            self.cache.extend(seq.seq_id, [token])
            scheduled.append(ScheduledSeq(seq, [token], 1))
            self.counters.decode_tokens += 1
            kept.append(seq)
        self.running = kept + queue + others
        return scheduled

    def _continue_prefills(self, now: float, budget: int) -> list[ScheduledSeq]:
        out: list[ScheduledSeq] = []
        pending = [s for s in self.running if not self._is_decoding(s) and self.cache.reserved_tokens(s.seq_id)
                   == self.cache.committed_tokens(s.seq_id)]
        pending.sort(key=lambda s: -self._score(s.admission_hit, s, now))
        for seq in pending:
            if budget <= 0:
                break
            remaining = self._remaining(seq)
            n = self._portion(remaining, budget)
            if not self.cache.can_extend(seq.seq_id, n):
                self.counters.stalled_portions += 1
                continue
            start = seq.num_tokens - remaining
            tokens = seq.all_token_ids[start:start + n]
            self.cache.extend(seq.seq_id, tokens)
            self.counters.prefill_tokens += n
            budget -= n
            out.append(ScheduledSeq(seq, tokens, self._samples_after(seq, n == remaining)))
        return out

    def _samples_after(self, seq: Sequence, reaches_end: bool) -> int:
        if not reaches_end:
            return 0
        return seq.params.n if (seq.params.n > 1 and not seq.output_token_ids) else 1

    def _preempt(self, seq: Sequence) -> None:
        self._nothing_admissible = False
        self.cache.release(seq.seq_id)
        seq.status = SequenceStatus.WAITING
        seq.num_preemptions += 1
        self.counters.preemptions += 1
        self.waiting.append(seq)

    def _admit(self, now: float, budget: int) -> list[ScheduledSeq]:
        admitted: list[ScheduledSeq] = []
        evaluated = budget > 0 and bool(self.waiting)
        owed_forks = 0                                   # forks of groups admitted earlier in this step
        for seq, cost, hit in self._ranked_waiting(now):
            if budget <= 0:
                break
            tokens = seq.all_token_ids
            if admitted:                                 # an earlier admission may have evicted what this hit counted on
                cost = self.cache.admission_cost(tokens)
                hit = self._hit(len(tokens), cost)
            first_of_group = seq.params.n > 1 and not seq.output_token_ids
            forks = seq.params.n - 1 if first_of_group else 0
            n = self._portion(cost.prefill_tokens, budget)
            fits = (
                len(self.running) + owed_forks + 1 + forks <= self.config.max_num_seqs
                and self.cache.fits(cost.pages_needed, owed_forks + forks + self.watermark_pages)
                and self.cache.free_state_slots() >= 1 + owed_forks + forks
            )
            if not fits:
                if now - seq.arrival_time >= self.config.max_skip_wait:
                    break
                continue
            ok = self.cache.admit(seq.seq_id, tokens, n)
            assert ok, "the fit check used a fresh cost"
            cached = self.cache.committed_tokens(seq.seq_id)
            fed = tokens[cached:cached + n]
            if seq.num_preemptions:
                self.counters.readmissions += 1
            else:
                self.counters.admissions += 1
            self.counters.cached_tokens += cached
            self.counters.prefill_tokens += len(fed)
            budget -= len(fed)
            owed_forks += forks
            seq.status = SequenceStatus.RUNNING
            seq.admission_hit = hit
            self.running.append(seq)
            admitted.append(ScheduledSeq(seq, fed, self._samples_after(seq, cached + len(fed) == len(tokens))))
        if admitted:
            chosen = {s.seq.seq_id for s in admitted}
            self.waiting = [s for s in self.waiting if s.seq_id not in chosen]
        self._nothing_admissible = evaluated and not admitted
        self._window_releases_seen = self.cache.counters.window_releases
        return admitted

    # ------------------------------------------------------------------ the step after the one under way
    def schedule_ahead(self, under_way: list[ScheduledSeq]) -> list[ScheduledSeq] | None:
        """
        The step that follows `under_way`, whose samples are not known yet; None where that step
        depends on them (then nothing is changed).  Otherwise `under_way` is committed here (its
        tokens are known, and whatever reads their keys is launched after it), each continuing
        sequence reserves one slot with PENDING_TOKEN as its token, and `postprocess` is told so.
        """
        alive = [s for s in under_way if s.seq.status is SequenceStatus.RUNNING]
        if any(s.num_samples != 1 for s in alive) or {s.seq.seq_id for s in alive} != {s.seq_id for s in self.running}:
            return None
        # the step under way produces output number len(outputs) + 1
        going_on = [s.seq for s in alive if len(s.seq.output_token_ids) + 1 < s.seq.params.max_tokens]
        if not going_on:
            return None
        # Requests that wait rule the step out unless none of them could be admitted into it anyway: nobody
        # reaches max_tokens in the step under way, and either the sequence cap is full or the last admission
        # pass found room for none of them and nothing has made room since.  A request that ends on an
        # end-of-sequence token then hands its place on one step later than it would have.
        if self.waiting:
            if len(going_on) < len(alive):
                return None
            blocked = self._nothing_admissible and self._window_releases_seen == self.cache.counters.window_releases
            if not blocked and len(self.running) < self.config.max_num_seqs:
                return None
        if not self.cache.fits(self.cache.pages_for_one_more_each([seq.seq_id for seq in going_on])):
            return None                          # someone has to give way: decided when the tokens are known
        for s in alive:
            self.cache.commit(s.seq.seq_id, len(s.token_ids))
        pending = [PENDING_TOKEN]
        ahead = []
        for seq in going_on:
            self.cache.extend(seq.seq_id, pending, checked=True)
            ahead.append(ScheduledSeq(seq, pending, 1))
        self.counters.decode_tokens += len(ahead)
        return ahead

    # ------------------------------------------------------------------ after the model ran
    def _fork(self, parent: Sequence, index: int) -> Sequence:
        child = Sequence(next(self._seq_ids), parent.request_id, parent.prompt_token_ids, parent.params,
                         parent.arrival_time, status=SequenceStatus.RUNNING, sample_index=index,
                         admission_hit=parent.admission_hit)
        self.cache.fork(parent.seq_id, child.seq_id)
        self.running.append(child)
        self.groups[parent.request_id].append(child)
        return child

    def _finish_reason(self, seq: Sequence, token: int) -> str | None:
        if token == self.config.eos_token_id and not seq.params.ignore_eos:
            return "eos"
        if len(seq.output_token_ids) >= seq.params.max_tokens:
            return "length"
        return None

    def postprocess(self, scheduled: list[ScheduledSeq], sampled: list[list[int]], now: float,
                    ahead: list[ScheduledSeq] | None = None) -> list[RequestOutput]:
        """
        Commits the step, forks groups after their first sampling step, records tokens, frees what
        finished.  `ahead` is what `schedule_ahead(scheduled)` returned: the step is committed
        already, and the sequences in `ahead` get their pending token filled in.  Samples of a
        sequence that finished while this step was launched ahead are dropped.
        """
        finished: list[Sequence] = []
        pending = {s.seq.seq_id for s in ahead} if ahead is not None else ()
        for (seq, token_ids, num_samples), tokens in zip(scheduled, sampled, strict=True):
            assert len(tokens) == num_samples
            if seq.status is SequenceStatus.FINISHED:
                continue
            if ahead is None:
                self.cache.commit(seq.seq_id, len(token_ids))
            elif seq.seq_id in pending:
                self.cache.amend_last(seq.seq_id, tokens[0])
            if num_samples == 0:
                continue
            samples = [seq] + [self._fork(seq, i) for i in range(1, num_samples)]
            for sample, token in zip(samples, tokens):
                sample.output_token_ids.append(token)
                if sample.first_token_time is None:
                    sample.first_token_time = now
                reason = self._finish_reason(sample, token)
                if reason is not None:
                    self.cache.release(sample.seq_id, drop_reserved=sample.seq_id in pending)
                    sample.status = SequenceStatus.FINISHED
                    sample.finish_reason = reason
                    sample.finish_time = now
                    finished.append(sample)
        if finished:
            done = {s.seq_id for s in finished}
            self.running = [s for s in self.running if s.seq_id not in done]
            self._nothing_admissible = False
        outputs = []
        for request_id in dict.fromkeys(s.request_id for s in finished):
            group = self.groups[request_id]
            if len(group) == group[0].params.n and all(s.status is SequenceStatus.FINISHED for s in group):
                outputs.append(RequestOutput(request_id, self.groups.pop(request_id)))
        return outputs

    def stats(self) -> SchedulerStats:
        return replace(self.counters, num_waiting=len(self.waiting), num_running=len(self.running))
