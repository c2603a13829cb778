"""
From a model folder to a model on the device, and from a model to its cache.

tinyserve-llm's loader (model/loader.py:73-95) picks the model class by config.json, builds it in
the target dtype on the device and fills it from the safetensors files; this does the same through
the architecture registry, the parts' tensor declarations and the engine's own safetensors reader.
"""

from __future__ import annotations

import torch

from tinyserve_llm_b200.cache.manager import CacheLayout, CacheManager, plan_layout
from tinyserve_llm_b200.cache.storage import DeviceCacheStorage
from tinyserve_llm_b200.config.registry import load_model_spec
from tinyserve_llm_b200.ops import get_ops
from tinyserve_llm_b200.parts.base import Runtime
from tinyserve_llm_b200.parts.model import DecoderModel, declared_tensors
from tinyserve_llm_b200.weights.loader import load_tensors
from tinyserve_llm_b200.weights.random_init import random_tensors

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def resolve_dtype(dtype: str | torch.dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype must be bfloat16 or float32, got {dtype}")
        return dtype
    try:
        return DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype must be one of {sorted(DTYPES)}, got {dtype!r}") from None


def require_cuda(device: str | torch.device = "cuda") -> torch.device:
    device = torch.device(device)
    if device.type != "cuda" or not torch.cuda.is_available():
        raise RuntimeError("tinyserve_llm_b200 runs on a CUDA device (sm_100a) only; there is no CPU path")
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    return device


def load_model(model_dir: str, dtype: str | torch.dtype = "bfloat16", device: str | torch.device = "cuda", *,
               random_weights_seed: int | None = None) -> DecoderModel:
    """
    The model of the folder, chosen by its config.json.  With `random_weights_seed` the folder needs
    only config.json: every declared tensor is drawn instead of read, with the generator and in the
    dtype `write_random_model` uses, so that one seed gives one model whichever way it is made (the
    draws run on the host, about ten seconds per billion weights, and go to the device tensor by tensor).
    """
    device = require_cuda(device)
    dtype = resolve_dtype(dtype)
    _, spec = load_model_spec(model_dir)
    declared = declared_tensors(spec)
    if random_weights_seed is None:
        tensors = load_tensors(model_dir, declared, optional=spec.optional_tensors,
                               ignored_suffixes=spec.ignored_suffixes, device=device)
    else:
        tensors = {name: t.to(device) for name, t in random_tensors(declared, random_weights_seed, dtype=torch.bfloat16)}
    with torch.cuda.device(device):
        return DecoderModel(spec, tensors, Runtime(dtype=dtype, device=device, ops=get_ops()))


def build_cache(model: DecoderModel, page_tokens: int, num_pages: int, *, caching: bool = True,
                num_state_slots: int = 0) -> tuple[CacheLayout, CacheManager, DeviceCacheStorage]:
    layout = plan_layout(model.cache_needs(), page_tokens)
    storage = DeviceCacheStorage(layout, num_pages, model.rt.dtype, model.rt.device, model.rt.ops,
                                 num_state_slots=num_state_slots)
    manager = CacheManager(layout, num_pages, storage, caching=caching, num_state_slots=num_state_slots)
    return layout, manager, storage
