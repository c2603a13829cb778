"""
Causal grouped-query attention over the paged cache.

Reference formulas: qkv = n . Wqkv^T, columns [q | k | v] (model/llama.py:198-209); rotary on q and
k before the cache write (:210); keys stored rotated, values raw (engine/model_runner.py:100-102);
scores = q.k * scale with query j of a sequence at position ctx - q_len + j seeing keys up to its
own position (attention/torch_paged.py:24-46); kv head j serves query heads j*g .. (j+1)*g - 1;
output projection (model/llama.py:212).
"""

from __future__ import annotations

import torch

from tinyserve_llm_b200.config.spec import AttentionSpec
from tinyserve_llm_b200.parts.base import KVNeed, Mixer, Runtime, TensorDecl, part_class, register_part
from tinyserve_llm_b200.parts.linear import Linear, fuse_rows


MAX_HEAD_DIM = 256      # csrc/attention_generic.cu, the kernel every size falls back to


@register_part("mixer", "attention")
class PagedAttention(Mixer):
    graph_safe = True

    @classmethod
    def validate(cls, spec: AttentionSpec) -> None:
        """Sizes no attention kernel takes are refused when the model is described or built, not at its first step."""
        if spec.num_kv_heads <= 0 or spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"num_heads={spec.num_heads} is not a multiple of num_kv_heads={spec.num_kv_heads}")
        if spec.head_dim <= 0 or spec.head_dim % 16 or spec.head_dim > MAX_HEAD_DIM:
            raise ValueError(f"head_dim={spec.head_dim} is not supported: the attention kernels take multiples of 16 "
                             f"up to {MAX_HEAD_DIM}")

    @classmethod
    def declare(cls, spec: AttentionSpec) -> dict[str, TensorDecl]:
        cls.validate(spec)
        q = spec.num_heads * spec.head_dim
        kv = spec.num_kv_heads * spec.head_dim
        return {
            "q_proj.weight": TensorDecl((q, spec.hidden_size)),
            "k_proj.weight": TensorDecl((kv, spec.hidden_size)),
            "v_proj.weight": TensorDecl((kv, spec.hidden_size)),
            "o_proj.weight": TensorDecl((spec.hidden_size, q)),
        }

    def __init__(self, spec: AttentionSpec, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        super().__init__(spec, tensors, rt)
        self.validate(spec)
        self.qkv = Linear(fuse_rows([tensors["q_proj.weight"], tensors["k_proj.weight"],
                                     tensors["v_proj.weight"]]), rt)
        self.out = Linear(tensors["o_proj.weight"], rt)
        self.position = None
        if spec.position is not None:
            self.position = part_class("position", spec.position)(spec.position, {}, rt)

    def kv_need(self) -> KVNeed:
        return KVNeed(self.spec.num_kv_heads, self.spec.head_dim, self.spec.window)

    def forward(self, x: torch.Tensor, ctx, binding) -> torch.Tensor:
        spec, ops = self.spec, self.rt.ops
        table = self.position.table if self.position is not None else None
        qkv = None
        if self.position is None or table is not None:          # a few tokens: projection, rotation and cache write in one kernel
            qkv = ops.linear_rope_store(x, self.qkv.weight, ctx, binding, table, spec.num_heads, spec.num_kv_heads,
                                        spec.head_dim)
        if qkv is None:
            qkv = self.qkv(x)                                   # [T, (nh + 2 nkv) * hd]
            if self.position is not None and table is None:     # a position part that edits q and k itself
                nq = spec.num_heads * spec.head_dim
                nk = spec.num_kv_heads * spec.head_dim
                self.position.apply(qkv[:, :nq], qkv[:, nq:nq + nk], ctx)
            ops.rope_store(qkv, ctx, binding, table, spec.num_heads, spec.num_kv_heads, spec.head_dim)
        o = ops.paged_attention(qkv, ctx, binding, spec.num_heads, spec.num_kv_heads, spec.head_dim,
                                spec.scale, spec.window)         # [T, nh * hd]
        return self.out(o)
