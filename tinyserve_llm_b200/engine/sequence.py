"""
Request-level types: sampling parameters and the scheduler's view of one sequence.

Names and meanings follow tinyserve-llm (scheduler/sequence.py:8-56): SamplingParams(max_tokens,
temperature, n, ignore_eos); a Sequence keeps its prompt, outputs, arrival time, admission-time
cache hit, preemption count and finish reason.  `sample_index` (which of a request's n samples this
is) is new: it keys the sampling noise so that a draw does not depend on the batch around it.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum, auto


@dataclass(frozen=True)
class SamplingParams:
    max_tokens: int = 256
    temperature: float = 1.0      # 0: greedy
    n: int = 1                    # parallel samples of the same prompt
    ignore_eos: bool = False


class SequenceStatus(Enum):
    WAITING = auto()
    RUNNING = auto()
    FINISHED = auto()


@dataclass
class Sequence:
    seq_id: int
    request_id: int
    prompt_token_ids: tuple[int, ...]
    params: SamplingParams
    arrival_time: float
    status: SequenceStatus = SequenceStatus.WAITING
    output_token_ids: list[int] = field(default_factory=list)
    sample_index: int = 0
    admission_hit: float = 0.0
    num_preemptions: int = 0
    first_token_time: float | None = None
    finish_time: float | None = None
    finish_reason: str | None = None          # "eos" or "length"

    @property
    def all_token_ids(self) -> list[int]:
        return [*self.prompt_token_ids, *self.output_token_ids]

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_token_ids) + len(self.output_token_ids)
