"""
Load a model folder's tensors by name and check them against what the model's parts declare.

Reference behaviour (model/loader.py:28-70): every model*.safetensors of the folder is read,
`rotary_emb.inv_freq` buffers are skipped, a tied checkpoint's `lm_head.weight` is skipped, and an
unfilled parameter raises.  Which names may be skipped comes with the model description, not from here.  Here every problem of the checkpoint (missing tensors, unexpected
tensors, wrong shapes) is gathered into one error.

Stored dtypes are kept: bfloat16 stays bfloat16, a tensor stored in 32-bit floats stays so, integer
tensors become int32 (float16 becomes bfloat16).  The parts convert to what they compute with.
"""

from __future__ import annotations

import glob
import os
from typing import Iterable, Mapping

import torch

from tinyserve_llm_b200.parts.base import TensorDecl
from tinyserve_llm_b200.weights.safetensors_io import SafetensorsError, SafetensorsFile

class CheckpointError(ValueError):
    """The checkpoint does not fit the model: lists missing, unexpected and misshapen tensors."""

    def __init__(self, model_dir: str, missing: list[str], unexpected: list[str],
                 wrong_shape: list[tuple[str, tuple[int, ...], tuple[int, ...]]],
                 duplicate: list[str] | None = None) -> None:
        self.missing = missing
        self.unexpected = unexpected
        self.wrong_shape = wrong_shape
        self.duplicate = duplicate or []
        lines = [f"checkpoint in {model_dir} does not fit the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): {missing}")
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): {unexpected}")
        if wrong_shape:
            shown = [f"{n}: stored {list(got)}, expected {list(want)}" for n, got, want in wrong_shape]
            lines.append(f"  wrong shapes ({len(wrong_shape)}): {shown}")
        if self.duplicate:
            lines.append(f"  stored in more than one file ({len(self.duplicate)}): {self.duplicate}")
        super().__init__("\n".join(lines))


def checkpoint_files(model_dir: str) -> list[str]:
    files = sorted(glob.glob(os.path.join(model_dir, "model*.safetensors")))
    if not files:
        raise FileNotFoundError(f"no model*.safetensors in {model_dir}")
    return files


def _kept_dtype(t: torch.Tensor) -> torch.Tensor:
    if t.dtype in (torch.bfloat16, torch.float32):
        return t
    if t.dtype in (torch.float16, torch.float64):
        return t.to(torch.bfloat16 if t.dtype == torch.float16 else torch.float32)
    if t.dtype in (torch.int64, torch.int16, torch.int8, torch.uint8, torch.bool):
        return t.to(torch.int32)
    return t


def load_tensors(model_dir: str, declared: Mapping[str, TensorDecl], *, optional: Iterable[str] = (),
                 ignored_suffixes: Iterable[str] = (), device: torch.device | str = "cpu") -> dict[str, torch.Tensor]:
    """
    {name: tensor on `device`} for every declared name.  `optional` names and names ending in one
    of `ignored_suffixes` are accepted and dropped when present; which they are is the model
    description's business (`ModelSpec.optional_tensors`, `ModelSpec.ignored_suffixes`).  Raises
    CheckpointError listing everything that is wrong at once.
    """
    optional = set(optional)
    ignored = tuple(ignored_suffixes)
    files = [SafetensorsFile(p) for p in checkpoint_files(model_dir)]
    try:
        where: dict[str, SafetensorsFile] = {}
        unexpected, duplicate = [], []
        wrong_shape: list[tuple[str, tuple[int, ...], tuple[int, ...]]] = []
        for f in files:
            for name, entry in f.entries.items():
                if (ignored and name.endswith(ignored)) or name in optional:
                    continue
                if name not in declared:
                    unexpected.append(name)
                    continue
                if name in where:
                    duplicate.append(name)
                    continue
                where[name] = f
                if tuple(declared[name].shape) != entry.shape:
                    wrong_shape.append((name, entry.shape, tuple(declared[name].shape)))
        missing = [n for n in declared if n not in where]
        if missing or unexpected or wrong_shape or duplicate:
            raise CheckpointError(model_dir, missing, sorted(unexpected), wrong_shape, duplicate)
        out = {}
        for name in declared:
            out[name] = _kept_dtype(where[name].tensor(name)).to(device)
        return out
    finally:
        for f in files:
            f.close()


__all__ = ["CheckpointError", "SafetensorsError", "checkpoint_files", "load_tensors"]
