"""
RMSNorm with the residual add fused in.

Reference formulas (model/llama.py:52-67): s = f32(x) + f32(residual); the carried residual is s
rounded to the activation dtype; y = s * rsqrt(mean(s^2) + eps) uses the unrounded sum; the output
is round(y) * weight, the weight multiply coming after the rounding.  Without a residual, x itself
starts the residual stream (model/llama.py:246-247).
"""

from __future__ import annotations

import torch

from tinyserve_llm_b200.config.spec import RMSNormSpec
from tinyserve_llm_b200.parts.base import Norm, Runtime, TensorDecl, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    graph_safe = True

    @classmethod
    def declare(cls, spec: RMSNormSpec) -> dict[str, TensorDecl]:
        return {"weight": TensorDecl((spec.size,), init="unit")}

    def __init__(self, spec: RMSNormSpec, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        super().__init__(spec, tensors, rt)
        w = tensors["weight"]
        # A weight stored in 32-bit floats stays so; the kernel takes either beside bf16 activations.
        keep = w.dtype if (w.dtype == torch.float32 or rt.dtype == torch.float32) else rt.dtype
        if rt.dtype == torch.float32:
            keep = torch.float32
        self.weight = w.to(device=rt.device, dtype=keep).contiguous()
        self.eps = float(spec.eps)

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None,
                rows: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
        return self.rt.ops.add_rmsnorm(x, residual, self.weight, self.eps, rows)

    def forward_embedded(self, table: torch.Tensor, ids: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        return self.rt.ops.embed_rmsnorm(table, ids, self.weight, self.eps)
