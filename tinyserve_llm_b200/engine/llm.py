"""
The Python entry point: LLM(model_path).generate(prompts, SamplingParams(...)).

Names and meanings of the options follow tinyserve-llm (engine/llm_engine.py:66-185,
engine/interface.py:28-32): SchedulerConfig, CacheConfig(block_size, caching, device), dtype,
num_blocks (None: sized from free device memory after a warm-up step), gpu_memory_utilization, seed,
load_tokenizer; add_request / step / generate; Completion and StepRecord.  There is no `attention`
option: the engine has one attention implementation, its own kernels.  New here: `cuda_graphs` and
`run_ahead` (decode steps launched before the previous step's samples have reached the host).
"""

from __future__ import annotations

import logging
import os
import time
from dataclasses import dataclass, replace

import torch

from tinyserve_llm_b200.cache.manager import PENDING_TOKEN, CacheStats, plan_layout
from tinyserve_llm_b200.cache.storage import DeviceCacheStorage
from tinyserve_llm_b200.engine.loading import build_cache, load_model, require_cuda, resolve_dtype
from tinyserve_llm_b200.engine.scheduler import RequestOutput, ScheduledSeq, Scheduler, SchedulerConfig, SchedulerStats
from tinyserve_llm_b200.engine.sequence import SamplingParams, SequenceStatus
from tinyserve_llm_b200.engine.step import GRAPH_MAX_TOKENS, StepEntry, StepRunner, StepShape
from tinyserve_llm_b200.sampling.sampler import PendingTokens, Sampler

logger = logging.getLogger(__name__)


@dataclass(frozen=True)
class CacheConfig:
    block_size: int = 256        # tokens per cache page
    caching: bool = True         # False turns prefix reuse off; forks still share pages
    device: str = "cuda"


def pages_that_fit(total: int, free: int, utilisation: float, step_peak: int, graphs_held: int, bytes_per_page: int) -> int:
    """
    Pages the pool may have: `utilisation` x the device's memory, less what is in use already (the
    weights, other processes), less the largest step's activations, less what decode graphs keep
    for good, in whole pages.  Zero or less means the engine does not fit.
    """
    budget = total * utilisation - (total - free) - step_peak - graphs_held
    return int(budget // max(bytes_per_page, 1))


@dataclass
class StepRecord:
    """One engine step; the two stats are running totals (subtract consecutive records)."""

    start: float
    end: float
    num_seqs: int
    num_tokens: int
    scheduler: SchedulerStats
    cache: CacheStats


@dataclass
class Completion:
    """A finished request: its n samples in fork order."""

    request_id: int
    prompt_token_ids: list[int]
    token_ids: list[list[int]]
    texts: list[str] | None
    finish_reasons: list[str]
    arrival_time: float
    first_token_time: float
    finish_time: float


@dataclass
class _InFlight:
    """A step that has been queued on the device."""

    batch: list[ScheduledSeq]
    pending: PendingTokens
    first_draw: dict[int, int]        # sequence id -> index of its first sample among the step's samples


class LLM:
    def __init__(
            self,
            model_path: str,
            scheduler_config: SchedulerConfig = SchedulerConfig(),
            cache_config: CacheConfig = CacheConfig(),
            *,
            dtype: torch.dtype | str = torch.bfloat16,
            num_blocks: int | None = None,
            gpu_memory_utilization: float = 0.9,
            seed: int | None = None,
            load_tokenizer: bool | None = None,
            random_weights_seed: int | None = None,
            cuda_graphs: bool = True,
            run_ahead: bool = True,
    ) -> None:
        self.device = require_cuda(cache_config.device)
        self.dtype = resolve_dtype(dtype)
        torch.cuda.set_device(self.device)
        self.model = load_model(model_path, self.dtype, self.device, random_weights_seed=random_weights_seed)
        spec = self.model.spec
        if scheduler_config.max_model_len > spec.max_positions:
            raise ValueError(f"max_model_len = {scheduler_config.max_model_len} exceeds the model's "
                             f"max_position_embeddings = {spec.max_positions}")
        self.tokenizer = None
        if load_tokenizer is None:
            load_tokenizer = any(os.path.isfile(os.path.join(model_path, f))
                                 for f in ("tokenizer.json", "tokenizer.model", "tokenizer_config.json"))
        if load_tokenizer:
            from transformers import AutoTokenizer          # text <-> ids only; no model code
            self.tokenizer = AutoTokenizer.from_pretrained(model_path)
        if scheduler_config.eos_token_id == -1:
            scheduler_config = replace(scheduler_config, eos_token_id=self._eos_token_id())
        self.scheduler_config = scheduler_config
        self.cache_config = cache_config
        needs_state = any(state for _, state in self.model.cache_needs())
        state_slots = scheduler_config.max_num_seqs if needs_state else 0
        if num_blocks is None:
            num_blocks = self._size_cache(gpu_memory_utilization, state_slots, cuda_graphs)
        self.layout, self.cache, self.storage = build_cache(
            self.model, cache_config.block_size, num_blocks, caching=cache_config.caching, num_state_slots=state_slots)
        self.scheduler = Scheduler(scheduler_config, self.cache)
        self.runner = StepRunner(self.model, self.cache, self.storage, cuda_graphs=cuda_graphs,
                                 max_model_len=scheduler_config.max_model_len,
                                 max_decode_batch=scheduler_config.max_num_seqs)
        self.sampler = Sampler(self.model.rt.ops, self.device, seed)
        self.steps: list[StepRecord] = []
        self.run_ahead = bool(run_ahead)
        self._in_flight: _InFlight | None = None
        self.steps_launched_ahead = 0
        logger.info("cache: %d pages of %d tokens", num_blocks, cache_config.block_size)

    # ------------------------------------------------------------------ set-up helpers
    def _eos_token_id(self) -> int:
        if self.tokenizer is not None and self.tokenizer.eos_token_id is not None:
            return int(self.tokenizer.eos_token_id)
        return self.model.spec.eos_token_id

    def _size_cache(self, utilisation: float, state_slots: int, cuda_graphs: bool) -> int:
        """
        Measures what the engine itself will need at its worst and gives the page pool the rest of
        `utilisation` x the device's memory.  tinyserve-llm warms up with the token budget spread
        over as many sequences as the cap allows, every one sampling, so that the [rows, vocab]
        logits and the sampler's buffers are in the measured peak (engine/llm_engine.py:112-140).
        The same step runs here, on a throwaway pool.  Then, where steps will be replayed from
        CUDA graphs, the widest ones the configuration allows (every sequence slot taken, block
        tables for `max_model_len`; once decoding, once beside the longest prompt portion a graph
        takes) are captured: what the graphs hold (their shared logits buffer and their memory
        pool, which the widest graphs size) stays allocated beside every later step.
        """
        cfg, page = self.scheduler_config, self.cache_config.block_size
        device = self.device
        seqs = min(cfg.max_num_seqs, cfg.max_num_batched_tokens)
        each = max(1, min(cfg.max_num_batched_tokens // seqs, cfg.max_model_len - 1, cfg.prefill_chunk or (1 << 30)))
        limit = GRAPH_MAX_TOKENS                                            # the largest step with a portion that a graph takes
        portion = max(0, min(limit - (seqs - 1), cfg.max_model_len - each - 3, cfg.prefill_chunk or limit))
        pages = seqs * -(-(each + 2) // page) + -(-portion // page) + 2
        _, manager, storage = build_cache(self.model, page, pages, caching=False, num_state_slots=max(state_slots, 1))
        eager = StepRunner(self.model, manager, storage, cuda_graphs=False)
        sampler = Sampler(self.model.rt.ops, device, 0)
        torch.cuda.synchronize(device)
        torch.cuda.reset_peak_memory_stats(device)
        baseline = torch.cuda.memory_allocated(device)
        entries = [StepEntry(i, [0] * each, [each - 1]) for i in range(seqs)]
        for e in entries:
            manager.admit(e.seq_id, e.tokens)
        logits = eager.step(entries)
        sampler.sample_async(logits, [1.0] * seqs, [(i, 0, 0) for i in range(seqs)]).wait()
        torch.cuda.synchronize(device)
        step_peak = torch.cuda.max_memory_allocated(device) - baseline
        del logits, sampler
        for e in entries:
            manager.commit(e.seq_id, each)
            manager.extend(e.seq_id, [0])
        # One decode step for every batch size a graph will be captured for, beyond those the engine's own product
        # serves: the library picks and loads its kernels per row count at first use (tens to hundreds of
        # milliseconds), which would otherwise fall on the first step of that size while requests wait.
        rows = 2 * self.model.rt.ops.skinny_max_rows
        while rows <= StepRunner.bucket(seqs):
            eager.step([StepEntry(i, [0], [0]) for i in range(min(rows, seqs))])
            rows *= 2
        torch.cuda.synchronize(device)
        del eager
        graphs_held = 0
        if cuda_graphs and self.model.graph_safe:
            torch.cuda.empty_cache()
            before = torch.cuda.memory_reserved(device)
            widest = [-(-cfg.max_model_len // page)] * len(manager.pools)
            replayed = StepRunner(self.model, manager, storage, max_model_len=cfg.max_model_len,
                                  max_decode_batch=cfg.max_num_seqs, table_pages=widest)
            widest_tables = tuple(replayed._graph_widths)
            batch = StepRunner.bucket(seqs)
            replayed._capture([StepEntry(i, [0], [0]) for i in range(seqs)], StepShape(batch, batch, 0, 1, True, widest_tables))
            if portion > 1:
                # ... and the largest step with a prompt portion that is replayed from a graph
                mixed = []
                for i in range(seqs):
                    manager.commit(i, 1)
                    fed = [0] * (portion if i == 0 else 1)
                    manager.extend(i, fed)
                    mixed.append(StepEntry(i, fed, [len(fed) - 1]))
                shape = replayed.graph_shape(mixed)
                if shape is not None:
                    replayed._capture(mixed, StepShape(shape.tokens, shape.seqs, shape.portions, shape.max_q, seqs > 1,
                                                       widest_tables))
            torch.cuda.synchronize(device)
            torch.cuda.empty_cache()             # what the capture's eager run cached goes; what the graphs hold stays
            graphs_held = max(0, torch.cuda.memory_reserved(device) - before)
            del replayed
        del manager, storage, entries
        torch.cuda.empty_cache()
        free, total = torch.cuda.mem_get_info(device)
        layout = plan_layout(self.model.cache_needs(), page)
        per_page = sum(DeviceCacheStorage.bytes_per_page(layout, self.dtype))
        num_blocks = pages_that_fit(total, free, utilisation, step_peak, graphs_held, per_page)
        logger.info("warm-up: %d sequences of %d tokens, step peak %.2f GiB, decode graphs hold %.2f GiB", seqs, each,
                    step_peak / 2 ** 30, graphs_held / 2 ** 30)
        if num_blocks <= 0:
            raise RuntimeError("no memory left for the cache; lower max_num_batched_tokens or max_num_seqs, or raise "
                               "gpu_memory_utilization")
        return num_blocks

    # ------------------------------------------------------------------ the loop
    def add_request(self, prompt: str | list[int], params: SamplingParams = SamplingParams(),
                    arrival_time: float | None = None) -> int:
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("a text prompt needs a tokenizer; pass token ids or load_tokenizer=True")
            token_ids = self.tokenizer.encode(prompt)
        else:
            token_ids = [int(t) for t in prompt]
        vocab = self.model.spec.vocab_size
        if any(t < 0 or t >= vocab for t in token_ids):
            raise ValueError(f"prompt holds token ids outside the vocabulary of {vocab}")
        return self.scheduler.add_request(token_ids, params, time.perf_counter() if arrival_time is None else arrival_time)

    def _launch(self, batch: list[ScheduledSeq], before: "_InFlight | None" = None) -> "_InFlight":
        """
        Queues the step and its sampling on the device; nothing waits.  With `before` (the step
        under way, whose samples the host has not seen) an entry that feeds the unknown token gets
        that step's sample for the same sequence, passed on the device, and its output position is
        one further on; entries that feed a prompt portion are as ever.
        """
        entries, temperatures, draws, rows = [], [], [], []
        first_draw: dict[int, int] = {}
        row = 0
        for seq, fed, num_samples in batch:
            lag = 1 if (before is not None and fed[0] == PENDING_TOKEN) else 0
            if lag:
                entries.append(StepEntry(seq.seq_id, (0,), (0,) if num_samples else (), feed=before.first_draw[seq.seq_id]))
            else:
                entries.append(StepEntry(seq.seq_id, fed, [len(fed) - 1] if num_samples else []))
            first_draw[seq.seq_id] = len(draws)
            for i in range(num_samples):
                index = seq.sample_index if num_samples == 1 else i
                temperatures.append(seq.params.temperature)
                draws.append((seq.request_id, index, len(seq.output_token_ids) + lag))
                rows.append(row)
            row += 1 if num_samples else 0
        logits = self.runner.step(entries, None if before is None else before.pending.device_tokens)
        pending = self.sampler.sample_async(logits, temperatures, draws, rows)
        return _InFlight(batch, pending, first_draw)

    def step(self) -> list[RequestOutput]:
        """
        One step's results.  With `run_ahead`, the step after it is launched before this one's
        samples are read where the scheduler can decide it without them, so the device does not
        idle while the host books the results; what `step()` returns, and when a request counts
        as finished, is the same either way.
        """
        start = time.perf_counter()
        flight = self._in_flight
        self._in_flight = None
        if flight is None:
            batch = self.scheduler.schedule(start)
            if not batch:
                raise RuntimeError("the scheduler produced an empty step")
            flight = self._launch(batch)
        ahead = self.scheduler.schedule_ahead(flight.batch) if self.run_ahead else None
        following = self._launch(ahead, flight) if ahead is not None else None
        self.steps_launched_ahead += ahead is not None
        tokens = flight.pending.wait()
        sampled, i = [], 0
        for _, _, num_samples in flight.batch:
            sampled.append(tokens[i:i + num_samples])
            i += num_samples
        end = time.perf_counter()
        outputs = self.scheduler.postprocess(flight.batch, sampled, end, ahead)
        if following is not None and any(s.seq.status is SequenceStatus.RUNNING for s in following.batch):
            self._in_flight = following          # else every sequence in it has finished: its results are dropped
        self.steps.append(StepRecord(start, end, len(flight.batch), sum(len(fed) for _, fed, _ in flight.batch),
                                     self.scheduler.stats(), self.cache.stats()))
        return outputs

    def generate(self, prompts: list[str] | list[list[int]],
                 params: SamplingParams | list[SamplingParams] = SamplingParams()) -> list[Completion]:
        """Runs the prompts to completion; results come back in prompt order."""
        params = params if isinstance(params, list) else [params] * len(prompts)
        if len(params) != len(prompts):
            raise ValueError(f"{len(prompts)} prompts but {len(params)} sampling parameter sets")
        order = [self.add_request(p, sp) for p, sp in zip(prompts, params)]
        done: dict[int, RequestOutput] = {}
        while self.scheduler.has_unfinished():
            for output in self.step():
                done[output.request_id] = output
        return [self._completion(done[r]) for r in order]

    def _completion(self, output: RequestOutput) -> Completion:
        seqs = sorted(output.sequences, key=lambda s: s.sample_index)
        token_ids = [list(s.output_token_ids) for s in seqs]
        texts = None
        if self.tokenizer is not None:
            texts = [self.tokenizer.decode(t, skip_special_tokens=True) for t in token_ids]
        return Completion(
            request_id=output.request_id,
            prompt_token_ids=list(seqs[0].prompt_token_ids),
            token_ids=token_ids,
            texts=texts,
            finish_reasons=[s.finish_reason for s in seqs],
            arrival_time=seqs[0].arrival_time,
            first_token_time=min(s.first_token_time for s in seqs),
            finish_time=max(s.finish_time for s in seqs),
        )
