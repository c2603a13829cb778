"""
Token sampling: greedy at temperature 0, otherwise a draw from softmax(logits / temperature).

tinyserve-llm draws with the Gumbel-max trick in exponential form from one generator stream for
the whole batch (engine/sampler.py:13-23).  Here the kernel uses counter-based noise keyed per draw
by (seed, request, sample index, output position), so a request's tokens do not depend on what
else is in the batch or on how its prompt was cut into portions.
"""

from __future__ import annotations

from typing import Sequence

import numpy as np
import torch

_GOLDEN = np.uint64(0x9E3779B97F4A7C15)
_FIELD_SALT = [np.uint64((0x9E3779B97F4A7C15 * (c + 2)) & 0xFFFFFFFFFFFFFFFF) for c in range(3)]
_MUL_A = np.uint64(0xBF58476D1CE4E5B9)
_MUL_B = np.uint64(0x94D049BB133111EB)


def _mix(z: np.ndarray) -> np.ndarray:
    """The finaliser of splitmix64 on an array of uint64 (arithmetic wraps)."""
    z = (z ^ (z >> np.uint64(30))) * _MUL_A
    z = (z ^ (z >> np.uint64(27))) * _MUL_B
    return z ^ (z >> np.uint64(31))


def draw_keys(seed: int, draws) -> np.ndarray:
    """
    int32 [n, 2]: the two words of the kernel's Philox key for each draw (request id, sample index,
    output position), a chain of splitmix64 finalisers over the seed and the three fields.  One
    vectorised pass: a step of hundreds of requests spends microseconds here, not a hash call each.
    """
    fields = np.asarray(draws, dtype=np.int64).reshape(-1, 3).astype(np.uint64)
    h = _mix(np.full(fields.shape[0], seed, dtype=np.int64).astype(np.uint64) + _GOLDEN)
    for c in range(3):
        h = _mix(h ^ (fields[:, c] + _FIELD_SALT[c]))
    return h.view(np.int32).reshape(-1, 2)


def draw_key(seed: int, request_id: int, sample_index: int, position: int) -> tuple[int, int]:
    """Two 32-bit words for the kernel's Philox key."""
    k0, k1 = draw_keys(seed, [(request_id, sample_index, position)])[0]
    return int(k0), int(k1)


class PendingTokens:
    """A step's samples: on the device at once, on the host after `wait()`."""

    def __init__(self, device_tokens: torch.Tensor | None, host: torch.Tensor | None, ready: torch.cuda.Event | None,
                 count: int) -> None:
        self.device_tokens = device_tokens      # int32 [count]; feeds the next step without a trip to the host
        self._host = host
        self._ready = ready
        self.count = count
        self._tokens: list[int] | None = [] if count == 0 else None

    def wait(self) -> list[int]:
        """Python ints: the step's one device-to-host read."""
        if self._tokens is None:
            self._ready.synchronize()
            self._tokens = self._host[:self.count].tolist()
        return self._tokens


class Sampler:
    SLOTS = 3          # pinned result buffers in rotation: a result is read before its buffer comes round again

    def __init__(self, ops, device: torch.device, seed: int | None = None) -> None:
        self.ops = ops
        self.device = device
        if seed is None:
            seed = int.from_bytes(__import__("os").urandom(7), "little")
        self.seed = int(seed)
        self._results: list[torch.Tensor | None] = [None] * self.SLOTS
        self._inputs: list[torch.Tensor | None] = [None] * self.SLOTS     # pinned too: temperatures and keys on their way up
        self._turn = 0

    def sample(self, logits: torch.Tensor, temperatures: Sequence[float], draws: Sequence[tuple[int, int, int]],
               rows: Sequence[int] | None = None) -> list[int]:
        """One token per draw, as Python ints; see `sample_async`."""
        return self.sample_async(logits, temperatures, draws, rows).wait()

    def sample_async(self, logits: torch.Tensor, temperatures: Sequence[float], draws: Sequence[tuple[int, int, int]],
                     rows: Sequence[int] | None = None) -> PendingTokens:
        """
        One token per draw.  `logits` is float32 [R, vocab]; draw i uses logits row rows[i] (default
        row i), temperature temperatures[i] and noise keyed by draws[i] = (request id, sample index,
        output position).  The kernel and the copy to pinned host memory are queued; nothing waits.
        At most SLOTS - 1 results may be outstanding when the next one is asked for.
        """
        count = len(draws)
        if count == 0:
            return PendingTokens(None, None, None, 0)
        if rows is not None and list(rows) != list(range(logits.shape[0])):
            logits = logits.index_select(0, torch.tensor(list(rows), dtype=torch.int64, device=logits.device))
        temps = np.asarray(temperatures, dtype=np.float32)
        keys = draw_keys(self.seed, draws)
        keys[temps <= 0] = 0                               # greedy rows draw nothing
        slot = self._turn
        self._turn = (slot + 1) % self.SLOTS
        staged = self._inputs[slot]                        # its last copy has run: that step's result has been read since
        if staged is None or staged.numel() < 3 * count:
            staged = self._inputs[slot] = torch.empty(max(3 * count, 192), dtype=torch.int32).pin_memory()
        packed = staged.numpy()
        packed[:count] = temps.view(np.int32)
        packed[count:3 * count] = keys.reshape(-1)
        dev = staged[:3 * count].to(self.device, non_blocking=True)                                # one small copy
        temps_dev = dev[:count].view(torch.float32)
        keys_dev = dev[count:].view(count, 2)
        tokens = self.ops.sample(logits.contiguous(), temps_dev, keys_dev)
        host = self._results[slot]
        if host is None or host.numel() < count:
            host = self._results[slot] = torch.empty(max(count, 64), dtype=torch.int32).pin_memory()
        host[:count].copy_(tokens, non_blocking=True)
        ready = torch.cuda.Event()
        ready.record()
        return PendingTokens(tokens, host, ready, count)
