"""Safetensors reading and writing, checkpoint errors, random-weights mode (no GPU)."""

import json
import os

import pytest
import torch
from safetensors import safe_open
from safetensors.torch import save_file

from tiny_configs import SEED_A, TINY_A, TINY_B, WEIGHTS
from tinyserve_llm_b200.config import LlamaConfig, llama_model_spec
from tinyserve_llm_b200.parts.model import declared_tensors
from tinyserve_llm_b200.weights import (CheckpointError, SafetensorsError, SafetensorsFile, load_tensors,
                                        random_tensors, write_random_model, write_safetensors)


def _declared(raw):
    spec = llama_model_spec(LlamaConfig.from_dict(raw))
    return spec, declared_tensors(spec)


def test_own_writer_is_read_by_the_safetensors_package_and_back(tmp_path):
    tensors = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.arange(7, dtype=torch.int64),
               "c": torch.randn(2, 2, 2), "d": torch.tensor(3.5)}
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, tensors, {"k": "v"})
    with safe_open(path, "pt", "cpu") as f:
        assert set(f.keys()) == set(tensors)
        for k in tensors:
            assert torch.equal(f.get_tensor(k), tensors[k])
    theirs = str(tmp_path / "y.safetensors")
    save_file(tensors, theirs)
    with SafetensorsFile(theirs) as f:
        for k in tensors:
            assert torch.equal(f.tensor(k), tensors[k]) and f.entries[k].dtype == tensors[k].dtype


def test_random_model_loads_and_keeps_stored_dtypes(tmp_path):
    folder = str(tmp_path)
    write_random_model(folder, TINY_A, SEED_A, **WEIGHTS)
    assert json.load(open(os.path.join(folder, "config.json"))) == TINY_A
    spec, declared = _declared(TINY_A)
    tensors = load_tensors(folder, declared, optional=spec.optional_tensors, ignored_suffixes=spec.ignored_suffixes)
    assert set(tensors) == set(declared)
    assert all(t.dtype == torch.bfloat16 for t in tensors.values())
    write_random_model(folder, TINY_A, SEED_A, store_dtype="float32", **WEIGHTS)
    again = load_tensors(folder, declared)
    assert all(t.dtype == torch.float32 for t in again.values())       # stored in 32-bit stays 32-bit
    for k in tensors:                                                     # same draws, rounded once
        assert torch.equal(again[k].to(torch.bfloat16), tensors[k])
    norm = again["model.layers.0.input_layernorm.weight"]
    assert abs(norm.mean().item() - 1.0) < 0.2 and norm.std().item() > 0.1


def test_random_values_depend_on_seed_and_name_only():
    _, declared = _declared(TINY_A)
    first = dict(random_tensors(declared, 5))
    reordered = dict(random_tensors(dict(reversed(list(declared.items()))), 5))
    other = dict(random_tensors(declared, 6))
    for k in declared:
        assert torch.equal(first[k], reordered[k])
    assert not torch.equal(first["model.norm.weight"], other["model.norm.weight"])


def test_integer_tables_become_int32_and_sharded_checkpoints_load(tmp_path):
    spec, declared = _declared(TINY_A)
    tensors = dict(random_tensors(declared, 1))
    names = sorted(tensors)
    half = len(names) // 2
    save_file({k: tensors[k] for k in names[:half]}, str(tmp_path / "model-00001-of-00002.safetensors"))
    second = {k: tensors[k] for k in names[half:]}
    second["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.ones(8)     # old checkpoints carry it: skipped
    second["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()    # tied copy: accepted and dropped
    save_file(second, str(tmp_path / "model-00002-of-00002.safetensors"))
    loaded = load_tensors(str(tmp_path), declared, optional=spec.optional_tensors, ignored_suffixes=spec.ignored_suffixes)
    assert all(torch.equal(loaded[k], tensors[k]) for k in tensors)
    from tinyserve_llm_b200.parts.base import TensorDecl
    save_file({"table": torch.arange(6, dtype=torch.int64).reshape(2, 3)}, str(tmp_path / "model.safetensors"))
    os.remove(tmp_path / "model-00001-of-00002.safetensors"), os.remove(tmp_path / "model-00002-of-00002.safetensors")
    table = load_tensors(str(tmp_path), {"table": TensorDecl((2, 3))})["table"]
    assert table.dtype == torch.int32 and table.tolist() == [[0, 1, 2], [3, 4, 5]]


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    spec, declared = _declared(TINY_B)
    tensors = dict(random_tensors(declared, 2))
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["lm_head.weight"]
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(5, 5, dtype=torch.bfloat16)
    tensors["model.layers.9.mlp.down_proj.weight"] = torch.zeros(2, 2)
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(2)
    save_file(tensors, str(tmp_path / "model.safetensors"))
    with pytest.raises(CheckpointError) as err:
        load_tensors(str(tmp_path), declared, optional=spec.optional_tensors, ignored_suffixes=spec.ignored_suffixes)
    e = err.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "lm_head.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.q_proj.bias", "model.layers.9.mlp.down_proj.weight"]
    assert e.wrong_shape == [("model.layers.0.self_attn.q_proj.weight", (5, 5), (192, 192))]
    text = str(e)
    assert "missing tensors (2)" in text and "unexpected tensors (2)" in text and "wrong shapes (1)" in text
    assert "stored [5, 5], expected [192, 192]" in text


def test_untied_model_does_not_accept_a_missing_head(tmp_path):
    spec, declared = _declared(TINY_B)
    tensors = dict(random_tensors(declared, 2))
    del tensors["lm_head.weight"]
    save_file(tensors, str(tmp_path / "model.safetensors"))
    with pytest.raises(CheckpointError, match="lm_head.weight"):
        load_tensors(str(tmp_path), declared, optional=spec.optional_tensors, ignored_suffixes=spec.ignored_suffixes)


def test_no_files_and_truncated_files(tmp_path):
    _, declared = _declared(TINY_A)
    with pytest.raises(FileNotFoundError, match="model\\*.safetensors"):
        load_tensors(str(tmp_path), declared)
    write_random_model(str(tmp_path), TINY_A, 1)
    path = tmp_path / "model.safetensors"
    data = path.read_bytes()
    path.write_bytes(data[: len(data) // 2])
    with pytest.raises(SafetensorsError, match="truncated"):
        load_tensors(str(tmp_path), declared)
    path.write_bytes(data[:5])
    with pytest.raises(SafetensorsError, match="header"):
        load_tensors(str(tmp_path), declared)
