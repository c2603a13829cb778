"""
Arrangements: how a block wires its mixer, feed-forward and norms.

"pre_norm" is the reference's decoder layer (model/llama.py:238-253): the residual add is deferred
into the following norm, so a block takes and returns (branch output, residual stream).
"""

from __future__ import annotations

import torch

from tinyserve_llm_b200.config.spec import BlockSpec
from tinyserve_llm_b200.parts.base import Runtime, TensorDecl, part_class, register_arrangement


def _sub(tensors: dict[str, torch.Tensor], prefix: str) -> dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


@register_arrangement("pre_norm")
class PreNormBlock:
    """x = x + mixer(norm1(x)); x = x + ffn(norm2(x)), with both adds fused into the next norm."""

    takes_token_ids = True        # forward(..., embedding=table): x holds token ids, the first norm gathers the rows

    @classmethod
    def declare(cls, spec: BlockSpec) -> dict[str, TensorDecl]:
        """Names local to the block's prefix."""
        out: dict[str, TensorDecl] = {}
        for role, part, prefix in cls._members(spec):
            for name, decl in part_class(role, part).declare(part).items():
                out[prefix + name] = decl
        return out

    @staticmethod
    def _members(spec: BlockSpec):
        return (
            ("norm", spec.mixer_norm, spec.mixer_norm_prefix),
            ("mixer", spec.mixer, spec.mixer_prefix),
            ("norm", spec.feed_forward_norm, spec.feed_forward_norm_prefix),
            ("feed_forward", spec.feed_forward, spec.feed_forward_prefix),
        )

    def __init__(self, spec: BlockSpec, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        self.spec = spec
        built = [part_class(role, part)(part, _sub(tensors, prefix), rt)
                 for role, part, prefix in self._members(spec)]
        self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward = built

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None, ctx, binding, embedding: torch.Tensor | None = None):
        """`embedding`: this is the model's first block and `x` holds token ids, rows of that table."""
        if embedding is not None:
            x, residual = self.mixer_norm.forward_embedded(embedding, x)
        else:
            x, residual = self.mixer_norm.forward(x, residual)
        x = self.mixer.forward(x, ctx, binding)
        x, residual = self.feed_forward_norm.forward(x, residual)
        x = self.feed_forward.forward(x, ctx)
        return x, residual
