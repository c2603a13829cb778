"""
Random-weights mode: a model folder (config.json, model.safetensors) from a configuration and a seed.

The reference has no such mode in its package; its tests draw framework-default initial weights and
randomise the norm weights so a missed norm shows (tests/test_llama.py:55-63).  Here every tensor a
model's parts declare is drawn from a generator keyed on (seed, tensor name), so the values do not
depend on the order of generation or on which tensors exist beside it.
"""

from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Iterator, Mapping

import torch

from tinyserve_llm_b200.config.registry import resolve_architecture
from tinyserve_llm_b200.parts.base import TensorDecl
from tinyserve_llm_b200.weights.safetensors_io import write_safetensors

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


def random_tensors(declared: Mapping[str, TensorDecl], seed: int, *, std: float = 0.02, unit_std: float = 0.01,
                   dtype: torch.dtype = torch.bfloat16,
                   device: torch.device | str = "cpu") -> Iterator[tuple[str, torch.Tensor]]:
    """Yields (name, tensor) in declaration order; values are drawn in float32 and rounded to `dtype`."""
    device = torch.device(device)
    for name, decl in declared.items():
        gen = torch.Generator(device=device).manual_seed(_tensor_seed(seed, name))
        t = torch.empty(decl.shape, dtype=torch.float32, device=device).normal_(0.0, 1.0, generator=gen)
        if decl.init == "unit":
            t = 1.0 + unit_std * t
        elif decl.init == "normal":
            t = std * t
        else:
            raise ValueError(f"tensor {name!r}: unknown init {decl.init!r}")
        yield name, t.to(dtype)


def write_random_model(model_dir: str, raw_config: Mapping[str, Any], seed: int, *, std: float = 0.02,
                       unit_std: float = 0.01, store_dtype: str = "bfloat16") -> None:
    """
    Writes `model_dir/config.json` (the given config.json keys, verbatim) and
    `model_dir/model.safetensors` (every tensor the architecture's parts declare).
    """
    from tinyserve_llm_b200.parts.model import declared_tensors     # parts register on import

    if store_dtype not in _STORE:
        raise ValueError(f"store_dtype must be one of {sorted(_STORE)}, got {store_dtype!r}")
    arch = resolve_architecture(raw_config)
    spec = arch.spec(arch.parse(raw_config))
    declared = declared_tensors(spec)
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(dict(raw_config), f, indent=2)
    tensors = dict(random_tensors(declared, seed, std=std, unit_std=unit_std, dtype=_STORE[store_dtype]))
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed)})
