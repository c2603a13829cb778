"""
Dense gated feed-forward: down(act(gate(x)) * up(x)), gate and up fused into one projection whose
output columns are [gate | up].

Reference: model/llama.py:77-83 (silu(gate) * up), :215-225 (fused gate_up, down; no biases).
"""

from __future__ import annotations

import torch

from tinyserve_llm_b200.config.spec import GatedMLPSpec
from tinyserve_llm_b200.parts.base import FeedForward, Runtime, TensorDecl, register_part
from tinyserve_llm_b200.parts.linear import Linear, fuse_rows


@register_part("feed_forward", "gated_mlp")
class GatedMLP(FeedForward):
    graph_safe = True

    ACTIVATIONS = ("silu",)

    @classmethod
    def declare(cls, spec: GatedMLPSpec) -> dict[str, TensorDecl]:
        return {
            "gate_proj.weight": TensorDecl((spec.intermediate_size, spec.hidden_size)),
            "up_proj.weight": TensorDecl((spec.intermediate_size, spec.hidden_size)),
            "down_proj.weight": TensorDecl((spec.hidden_size, spec.intermediate_size)),
        }

    def __init__(self, spec: GatedMLPSpec, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        super().__init__(spec, tensors, rt)
        if spec.activation not in self.ACTIVATIONS:
            raise NotImplementedError(f"activation {spec.activation!r} is not supported; have {self.ACTIVATIONS}")
        self.gate_up = Linear(fuse_rows([tensors["gate_proj.weight"], tensors["up_proj.weight"]]), rt)
        self.down = Linear(tensors["down_proj.weight"], rt)

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        return self.down(self.rt.ops.linear_swiglu(x, self.gate_up.weight))
