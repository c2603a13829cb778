"""
One registry from an architecture's name (config.json `architectures[0]`, with `model_type` as
fallback) to its typed configuration and to the builder of its `ModelSpec`.

Reference behaviour: a dict from `model_type` to the model class, and NotImplementedError naming
what is available for anything else (model/loader.py:22-25, :85-86).
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Mapping

from tinyserve_llm_b200.config.llama import ConfigError, LlamaConfig, llama_model_spec
from tinyserve_llm_b200.config.spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str                                         # config.json architectures[0]
    model_type: str                                   # config.json model_type
    parse: Callable[[Mapping[str, Any]], Any]         # raw config.json -> typed configuration
    spec: Callable[[Any], ModelSpec]                  # typed configuration -> ModelSpec


ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(arch: Architecture) -> Architecture:
    ARCHITECTURES[arch.name] = arch
    return arch


register_architecture(Architecture("LlamaForCausalLM", "llama", LlamaConfig.from_dict, llama_model_spec))


def resolve_architecture(raw: Mapping[str, Any]) -> Architecture:
    names = raw.get("architectures") or []
    for name in names:
        if name in ARCHITECTURES:
            return ARCHITECTURES[name]
    model_type = raw.get("model_type")
    for arch in ARCHITECTURES.values():
        if model_type is not None and arch.model_type == model_type:
            return arch
    raise NotImplementedError(
        f"architecture {list(names) or model_type!r} is not supported; have {sorted(ARCHITECTURES)}")


def read_config_json(model_dir: str) -> dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"no config.json in {model_dir}")
    with open(path, "r", encoding="utf-8") as f:
        raw = json.load(f)
    if not isinstance(raw, dict):
        raise ConfigError(f"{path} does not hold a JSON object")
    return raw


def load_model_spec(model_dir: str) -> tuple[Any, ModelSpec]:
    """(typed configuration, ModelSpec) of the model folder, chosen by its config.json."""
    raw = read_config_json(model_dir)
    arch = resolve_architecture(raw)
    config = arch.parse(raw)
    return config, arch.spec(config)
