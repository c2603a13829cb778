"""
The decoder: token embedding, the run list of blocks, final norm, vocabulary projection.

Reference: model/llama.py:256-304.  The run list (ModelSpec.run) is data: it may name a block more
than once and may let an execution read the cache entry another execution writes.  Only the rows
whose logits are wanted go through the final norm and the vocabulary projection
(engine/model_runner.py:126-127).
"""

from __future__ import annotations

import torch

from tinyserve_llm_b200.config.spec import ModelSpec
from tinyserve_llm_b200.parts import attention, mlp, norm, rotary  # noqa: F401  (registration)
from tinyserve_llm_b200.parts.base import KVNeed, Runtime, TensorDecl, arrangement_class, part_class
from tinyserve_llm_b200.parts.block import _sub
from tinyserve_llm_b200.parts.linear import Linear


def declared_tensors(spec: ModelSpec) -> dict[str, TensorDecl]:
    """Every tensor the checkpoint must hold, by its full name."""
    out: dict[str, TensorDecl] = {spec.embedding_name: TensorDecl((spec.vocab_size, spec.hidden_size))}
    for block in spec.blocks:
        for name, decl in arrangement_class(block.arrangement).declare(block).items():
            out[block.prefix + name] = decl
    for name, decl in part_class("norm", spec.final_norm).declare(spec.final_norm).items():
        out[spec.final_norm_prefix + name] = decl
    if spec.lm_head_name is not None:
        out[spec.lm_head_name] = TensorDecl((spec.vocab_size, spec.hidden_size))
    return out


class DecoderModel:
    def __init__(self, spec: ModelSpec, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        self.spec = spec
        self.rt = rt
        self.embedding = tensors[spec.embedding_name].to(device=rt.device, dtype=rt.dtype).contiguous()
        self.blocks = [
            arrangement_class(b.arrangement)(b, _sub(tensors, b.prefix), rt) for b in spec.blocks
        ]
        self.final_norm = part_class("norm", spec.final_norm)(
            spec.final_norm, _sub(tensors, spec.final_norm_prefix), rt)
        if spec.lm_head_name is None:
            self.lm_head = Linear.__new__(Linear)            # tied: the embedding table is the weight
            self.lm_head.rt = rt
            self.lm_head.weight = self.embedding
            self.lm_head.out_features, self.lm_head.in_features = self.embedding.shape
        else:
            self.lm_head = Linear(tensors[spec.lm_head_name], rt)
        self._check_run_list()
        # A CUDA graph may replay the model only if no part runs host code that depends on the step.
        self.graph_safe = all(getattr(part, "graph_safe", False) for block in self.blocks
                              for part in (block.mixer, block.feed_forward, block.mixer_norm, block.feed_forward_norm))

    def _check_run_list(self) -> None:
        writers: dict[int, int] = {}
        for i, entry in enumerate(self.spec.run):
            if not 0 <= entry.block < len(self.blocks):
                raise ValueError(f"run entry {i} names block {entry.block}; the model has {len(self.blocks)}")
            if entry.writes_cache:
                if entry.cache_entry in writers:
                    raise ValueError(f"cache entry {entry.cache_entry} is written by run entries "
                                     f"{writers[entry.cache_entry]} and {i}")
                writers[entry.cache_entry] = i
        for i, entry in enumerate(self.spec.run):
            if not entry.writes_cache and writers.get(entry.cache_entry, len(self.spec.run)) > i:
                raise ValueError(f"run entry {i} reads cache entry {entry.cache_entry} before anything wrote it")
            need_a = self.blocks[entry.block].mixer.kv_need()
            need_b = self.blocks[self.spec.run[writers[entry.cache_entry]].block].mixer.kv_need()
            if need_a != need_b:
                raise ValueError(f"run entry {i} reads a cache entry of another geometry: {need_a} vs {need_b}")

    # what the cache manager sizes itself from
    def cache_needs(self) -> list[tuple[KVNeed | None, int]]:
        """Per cache entry: (paged key/value need or None, bytes of fixed-size per-request state)."""
        needs: list[tuple[KVNeed | None, int]] = [(None, 0)] * self.spec.num_cache_entries
        for entry in self.spec.run:
            if entry.writes_cache:
                mixer = self.blocks[entry.block].mixer
                needs[entry.cache_entry] = (mixer.kv_need(), int(mixer.state_bytes()))
        return needs

    def forward(self, ctx) -> tuple[torch.Tensor, torch.Tensor | None]:
        """Runs the step's tokens through the run list; returns (last branch output, residual stream)."""
        # an arrangement that takes the embedding table reads the token ids itself (its first norm gathers the rows)
        run = self.spec.run
        first = self.blocks[run[0].block] if run else None
        if first is not None and getattr(first, "takes_token_ids", False):
            x, residual = first.forward(ctx.token_ids, None, ctx, ctx.binding(run[0]), embedding=self.embedding)
            run = run[1:]
        else:
            x, residual = self.rt.ops.embedding(self.embedding, ctx.token_ids), None
        for entry in run:
            x, residual = self.blocks[entry.block].forward(x, residual, ctx, ctx.binding(entry))
        return x, residual

    def logits(self, x: torch.Tensor, residual: torch.Tensor | None, rows: torch.Tensor,
               out: torch.Tensor | None = None) -> torch.Tensor:
        """float32 [len(rows), vocab] (into `out` if given): final norm and vocabulary projection of the wanted rows only."""
        h, _ = self.final_norm.forward(x, residual, rows)
        return self.lm_head(h, out_dtype=torch.float32, out=out)
