"""
Architecture-neutral description of a decoder: what the engine builds a model from.

An architecture's typed configuration (for instance `LlamaConfig`) is turned by its registered
builder into a `ModelSpec`: a list of block definitions (each naming a mixer, a feed-forward, its
norms and an arrangement, every size and constant as a field) and a run list that says in which
order the blocks execute and which cache entry each execution uses.  Nothing below this file knows
which architecture it serves.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class PartSpec:
    """Base of every part description. `kind` selects the implementation in the part registry."""

    kind: str = field(init=False, default="")


@dataclass(frozen=True)
class Llama3Scaling:
    """Frequency rescaling of llama3-type rotary embeddings (reference: model/llama.py:107-128)."""

    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int


@dataclass(frozen=True)
class RotarySpec(PartSpec):
    """Rotate-half rotary position encoding applied to queries and keys."""

    kind: str = field(init=False, default="rotary")
    head_dim: int = 0
    theta: float = 10000.0
    max_positions: int = 0
    scaling: Llama3Scaling | None = None


@dataclass(frozen=True)
class RMSNormSpec(PartSpec):
    kind: str = field(init=False, default="rmsnorm")
    size: int = 0
    eps: float = 1e-6


@dataclass(frozen=True)
class AttentionSpec(PartSpec):
    """Causal grouped-query attention over a paged key/value cache."""

    kind: str = field(init=False, default="attention")
    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    scale: float = 0.0            # multiplies q.k before the softmax
    window: int = 0               # 0: every earlier key; w > 0: the last w keys, the query's own included
    position: PartSpec | None = None


@dataclass(frozen=True)
class GatedMLPSpec(PartSpec):
    """Dense gated feed-forward: down(act(gate(x)) * up(x))."""

    kind: str = field(init=False, default="gated_mlp")
    hidden_size: int = 0
    intermediate_size: int = 0
    activation: str = "silu"


@dataclass(frozen=True)
class BlockSpec:
    """
    One layer definition: its parts, how they are wired, and the checkpoint prefix its tensors
    live under.  `arrangement` picks the wiring (the registry of arrangements); "pre_norm" is
    x + mixer(norm(x)) followed by x + ffn(norm(x)) with the adds deferred into the next norm.
    """

    arrangement: str
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    prefix: str                      # e.g. "model.layers.3."
    mixer_prefix: str = "self_attn."
    feed_forward_prefix: str = "mlp."
    mixer_norm_prefix: str = "input_layernorm."
    feed_forward_norm_prefix: str = "post_attention_layernorm."


@dataclass(frozen=True)
class RunEntry:
    """
    One execution of a block.  `block` indexes `ModelSpec.blocks` (the same block may be named by
    several entries: shared weights).  `cache_entry` is the cache/state entry this execution uses;
    entries that share a `cache_entry` share keys and values, and only the one with `writes_cache`
    stores into it (the others read what it stored in the same step).
    """

    block: int
    cache_entry: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    blocks: tuple[BlockSpec, ...]
    run: tuple[RunEntry, ...]
    final_norm: PartSpec
    embedding_name: str
    final_norm_prefix: str
    lm_head_name: str | None         # None: tied to the embedding
    max_positions: int
    eos_token_id: int
    optional_tensors: tuple[str, ...] = ()     # names a checkpoint may carry that the model does not read
    ignored_suffixes: tuple[str, ...] = ()     # tensors whose names end so are skipped (buffers the model recomputes)
    extras: dict[str, Any] = field(default_factory=dict, compare=False)

    @property
    def num_cache_entries(self) -> int:
        return 1 + max((e.cache_entry for e in self.run), default=-1)
