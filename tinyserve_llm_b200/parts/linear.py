"""
Bias-free projection y = x . W^T with W stored [out_features, in_features] (the checkpoint layout).

bfloat16: the library matrix product (cuBLAS through torch.mm), as the reference does through
nn.Linear (model/llama.py:200-201, :220-221).  float32: the engine's own FFMA kernel, so that no
reduced-precision matrix mode can slip in and the reduction order of a row does not depend on what
else is in the batch.
"""

from __future__ import annotations

import torch

from tinyserve_llm_b200.parts.base import Runtime


def fuse_rows(tensors: list[torch.Tensor]) -> torch.Tensor:
    """Stack projections that share an input into one weight, rows in the order given."""
    return torch.cat(tensors, dim=0).contiguous()


class Linear:
    def __init__(self, weight: torch.Tensor, rt: Runtime) -> None:
        assert weight.dim() == 2
        self.rt = rt
        self.weight = weight.to(device=rt.device, dtype=rt.dtype).contiguous()
        self.out_features, self.in_features = self.weight.shape

    def __call__(self, x: torch.Tensor, out_dtype: torch.dtype | None = None,
                 out: torch.Tensor | None = None) -> torch.Tensor:
        return self.rt.ops.linear(x, self.weight, out_dtype=out_dtype, out=out)
