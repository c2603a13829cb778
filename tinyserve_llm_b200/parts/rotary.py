"""
Rotate-half rotary position encoding with optional llama3 frequency rescaling.

Reference formulas: inv_freq[i] = 1 / theta^(2i/d) in float32 (model/llama.py:148); llama3 rescaling
by wavelength bands (:107-128); angle[p, i] = float32(p) * inv_freq[i]; the table row of position p
is [cos(angle) | sin(angle)] (:157-160).  The table is built once on the host in float32, in that
order of operations, and the kernels gather rows of it by position.
"""

from __future__ import annotations

import math

import torch

from tinyserve_llm_b200.config.spec import Llama3Scaling, RotarySpec
from tinyserve_llm_b200.parts.base import PositionEncoding, Runtime, register_part


def inverse_frequencies(head_dim: int, theta: float, scaling: Llama3Scaling | None) -> torch.Tensor:
    """float32 [head_dim // 2]."""
    exponent = torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim
    inv_freq = 1.0 / (theta ** exponent)
    if scaling is None:
        return inv_freq
    window = scaling.original_max_position_embeddings
    longest_kept = window / scaling.low_freq_factor      # wavelengths above this are slowed by `factor`
    shortest_scaled = window / scaling.high_freq_factor  # wavelengths below this are left alone
    wavelength = 2 * math.pi / inv_freq
    slowed = torch.where(wavelength > longest_kept, inv_freq / scaling.factor, inv_freq)
    blend = (window / wavelength - scaling.low_freq_factor) / (scaling.high_freq_factor - scaling.low_freq_factor)
    blended = (1 - blend) * slowed / scaling.factor + blend * slowed
    in_band = (wavelength >= shortest_scaled) & (wavelength <= longest_kept)
    return torch.where(in_band, blended, slowed)


def cos_sin_table(spec: RotarySpec, num_positions: int | None = None) -> torch.Tensor:
    """float32 [positions, head_dim]: cos of the head_dim/2 angles, then their sin."""
    n = spec.max_positions if num_positions is None else num_positions
    inv_freq = inverse_frequencies(spec.head_dim, spec.theta, spec.scaling)
    angles = torch.outer(torch.arange(n, dtype=torch.float32), inv_freq)
    return torch.cat((angles.cos(), angles.sin()), dim=-1).contiguous()


@register_part("position", "rotary")
class Rotary(PositionEncoding):
    def __init__(self, spec: RotarySpec, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        super().__init__(spec, tensors, rt)
        key = ("rotary", spec)
        if key not in rt.shared:               # one table for all layers with the same settings
            rt.shared[key] = cos_sin_table(spec).to(rt.device)
        self.table = rt.shared[key]
