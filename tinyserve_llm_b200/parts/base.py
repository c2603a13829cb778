"""
Interfaces and registries of the parts a decoder block is put together from.

A part is built from (its spec, its tensors, the runtime) and knows nothing of the model around it:
every size and constant reaches it through its spec.  Implementations register themselves under a
role ("mixer", "feed_forward", "norm", "position") and the spec's `kind`; the way parts are wired
into a block registers under "arrangement".  A new part needs only `@register_part(role, kind)` on
a class with the interface below; nothing in the engine, the cache or the loader changes.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch

from tinyserve_llm_b200.config.spec import PartSpec


@dataclass(frozen=True)
class TensorDecl:
    """A tensor a part expects in the checkpoint, under a name local to the part's prefix."""

    shape: tuple[int, ...]
    init: str = "normal"      # random-weights mode: "normal" = N(0, std); "unit" = 1 + N(0, unit_std)


@dataclass(frozen=True)
class KVNeed:
    """What a mixer needs from the paged cache, per cache entry."""

    num_kv_heads: int
    head_dim: int
    window: int = 0           # 0: all keys are kept; w > 0: only the last w


@dataclass
class Runtime:
    """What a part computes with: the activation dtype, the device and the kernel library."""

    dtype: torch.dtype        # torch.bfloat16 (serving) or torch.float32 (true 32-bit path)
    device: torch.device
    ops: Any                  # tinyserve_llm_b200.ops.Ops
    shared: dict = field(default_factory=dict)   # buffers parts of one model share (position tables)


class Part:
    """Common base: declares tensors, is constructed from them."""

    role = ""
    graph_safe = False        # True: forward() launches the same kernels whatever the step holds (CUDA graphs)

    @classmethod
    def declare(cls, spec: PartSpec) -> dict[str, TensorDecl]:
        return {}

    def __init__(self, spec: PartSpec, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        self.spec = spec
        self.rt = rt


class Norm(Part):
    """forward(x, residual) -> (normalised, new_residual); residual None means x starts the stream."""

    role = "norm"

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None,
                rows: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
        raise NotImplementedError

    def forward_embedded(self, table: torch.Tensor, ids: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """
        The model's first norm: its input rows are table[ids], which start the residual stream.
        A norm whose kernel can gather overrides this and saves the separate embedding kernel.
        """
        return self.forward(self.rt.ops.embedding(table, ids), None)


class PositionEncoding(Part):
    """
    Either exposes `table` ([max_positions, rotary_dim] fp32: cos half then sin half), which the
    attention kernels apply while they store keys, or overrides `apply` to change q and k in place.
    """

    role = "position"
    table: torch.Tensor | None = None

    def apply(self, q: torch.Tensor, k: torch.Tensor, ctx: Any) -> None:
        return None


class Mixer(Part):
    """
    Token mixer.  `kv_need()` asks the cache manager for pages (None: no keys/values);
    `state_bytes()` asks for a fixed-size per-request state slot (0: none).  `forward` receives the
    step context and the binding of its cache entry (pages, block tables, state rows).
    """

    role = "mixer"

    def kv_need(self) -> KVNeed | None:
        return None

    def state_bytes(self) -> int:
        return 0

    def forward(self, x: torch.Tensor, ctx: Any, binding: Any) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    role = "feed_forward"

    def forward(self, x: torch.Tensor, ctx: Any) -> torch.Tensor:
        raise NotImplementedError


_PARTS: dict[tuple[str, str], type] = {}
_ARRANGEMENTS: dict[str, type] = {}


def register_part(role: str, kind: str) -> Callable[[type], type]:
    def deco(cls: type) -> type:
        _PARTS[(role, kind)] = cls
        return cls
    return deco


def register_arrangement(name: str) -> Callable[[type], type]:
    def deco(cls: type) -> type:
        _ARRANGEMENTS[name] = cls
        return cls
    return deco


def part_class(role: str, spec: PartSpec) -> type:
    try:
        return _PARTS[(role, spec.kind)]
    except KeyError:
        have = sorted(k for r, k in _PARTS if r == role)
        raise NotImplementedError(f"no {role} part of kind {spec.kind!r}; have {have}") from None


def arrangement_class(name: str) -> type:
    try:
        return _ARRANGEMENTS[name]
    except KeyError:
        raise NotImplementedError(f"no block arrangement {name!r}; have {sorted(_ARRANGEMENTS)}") from None
