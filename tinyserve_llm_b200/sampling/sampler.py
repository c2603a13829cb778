"""
Token sampling: greedy at temperature 0, otherwise a draw from softmax(logits / temperature).

tinyserve-llm draws with the Gumbel-max trick in exponential form from one generator stream for
the whole batch (engine/sampler.py:13-23).  Here the kernel uses counter-based noise keyed per draw
by (seed, request, sample index, output position), so a request's tokens do not depend on what
else is in the batch or on how its prompt was cut into portions.
"""

from __future__ import annotations

import hashlib
import struct
from typing import Sequence

import torch


def draw_key(seed: int, request_id: int, sample_index: int, position: int) -> tuple[int, int]:
    """Two 32-bit words for the kernel's Philox key."""
    digest = hashlib.blake2b(struct.pack("<qqqq", seed, request_id, sample_index, position), digest_size=8).digest()
    k0, k1 = struct.unpack("<ii", digest)
    return k0, k1


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
        bits, keys = [], []
        for d, t in zip(draws, temperatures):
            bits.append(struct.unpack("<i", struct.pack("<f", t))[0])
            keys.extend(draw_key(self.seed, *d) if t > 0 else (0, 0))
        dev = torch.tensor(bits + keys, dtype=torch.int32).to(self.device, non_blocking=True)   # one small copy
        temps_dev = dev[:count].view(torch.float32)
        keys_dev = dev[count:].view(count, 2)
        tokens = self.ops.sample(logits.contiguous(), temps_dev, keys_dev)
        slot = self._turn
        self._turn = (slot + 1) % self.SLOTS
        host = self._results[slot]
        if host is None or host.numel() < count:
            host = self._results[slot] = torch.empty(max(count, 64), dtype=torch.int32).pin_memory()
        host[:count].copy_(tokens, non_blocking=True)
        ready = torch.cuda.Event()
        ready.record()
        return PendingTokens(tokens, host, ready, count)
