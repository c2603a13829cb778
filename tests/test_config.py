"""Configuration and registry (no GPU)."""

import copy

import pytest

from tiny_configs import TINY_A, TINY_B, TINY_C
from tinyserve_llm_b200.config import (ConfigError, LlamaConfig, Llama3Scaling, llama_model_spec,
                                       resolve_architecture)


def test_reads_every_size_from_config_json():
    a, b, c = (LlamaConfig.from_dict(x) for x in (TINY_A, TINY_B, TINY_C))
    assert (a.head_dim, b.head_dim, c.head_dim) == (16, 32, 48)          # default H/nh, stated, stated != H/nh
    assert (a.num_key_value_heads, b.num_key_value_heads, c.num_key_value_heads) == (2, 2, 1)
    assert a.rope_scaling is None and a.rope_theta == 10000.0
    assert b.rope_scaling == Llama3Scaling(8.0, 1.0, 4.0, 64) and b.rope_theta == 500000.0
    assert c.rope_scaling == Llama3Scaling(4.0, 1.0, 2.0, 32) and c.rope_theta == 1000000.0   # rope_parameters spelling
    assert (a.rms_norm_eps, b.rms_norm_eps, c.rms_norm_eps) == (1e-5, 1e-6, 1e-4)
    assert (a.tie_word_embeddings, b.tie_word_embeddings, c.tie_word_embeddings) == (True, False, False)
    assert (a.eos_token_id, b.eos_token_id, c.eos_token_id) == (3, 7, -1)   # int, first of a list, absent


def test_defaults_and_spellings():
    raw = copy.deepcopy(TINY_A)
    del raw["num_key_value_heads"], raw["rope_theta"], raw["tie_word_embeddings"]
    cfg = LlamaConfig.from_dict(raw)
    assert cfg.num_key_value_heads == cfg.num_attention_heads
    assert cfg.rope_theta == 10000.0 and cfg.tie_word_embeddings is False
    raw["rope_scaling"] = {"type": "default"}
    assert LlamaConfig.from_dict(raw).rope_scaling is None
    raw["rope_scaling"] = {"rope_type": "llama3", "factor": 2.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0}
    assert LlamaConfig.from_dict(raw).rope_scaling.original_max_position_embeddings == raw["max_position_embeddings"]


@pytest.mark.parametrize("change, needle", [
    ({"attention_bias": True}, "attention_bias"),
    ({"mlp_bias": True}, "mlp_bias"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "yarn"),
    ({"num_key_value_heads": 3}, "num_key_value_heads"),
    ({"rms_norm_eps": 0}, "rms_norm_eps"),
    ({"vocab_size": -5}, "vocab_size"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 2.0}}, "low_freq_factor"),
])
def test_refuses_what_it_does_not_implement(change, needle):
    with pytest.raises(ConfigError, match=needle):
        LlamaConfig.from_dict({**TINY_A, **change})


def test_missing_keys_are_named():
    raw = {k: v for k, v in TINY_A.items() if k not in ("hidden_size", "rms_norm_eps")}
    with pytest.raises(ConfigError, match="hidden_size.*rms_norm_eps"):
        LlamaConfig.from_dict(raw)


def test_registry_by_architecture_then_model_type():
    assert resolve_architecture(TINY_A).name == "LlamaForCausalLM"
    assert resolve_architecture({"model_type": "llama"}).name == "LlamaForCausalLM"
    with pytest.raises(NotImplementedError, match="LlamaForCausalLM"):
        resolve_architecture({"architectures": ["MambaForCausalLM"], "model_type": "mamba"})


def test_model_spec_carries_every_constant_as_a_parameter():
    spec = llama_model_spec(LlamaConfig.from_dict(TINY_B))
    assert len(spec.blocks) == 3 and [e.block for e in spec.run] == [0, 1, 2]
    assert [e.cache_entry for e in spec.run] == [0, 1, 2] and all(e.writes_cache for e in spec.run)
    mixer = spec.blocks[0].mixer
    assert (mixer.num_heads, mixer.num_kv_heads, mixer.head_dim, mixer.window) == (6, 2, 32, 0)
    assert mixer.scale == 32 ** -0.5 and mixer.position.theta == 500000.0
    assert spec.blocks[1].feed_forward.intermediate_size == 512
    assert spec.blocks[2].mixer_norm.eps == 1e-6 and spec.final_norm.eps == 1e-6
    assert spec.lm_head_name == "lm_head.weight"
    assert llama_model_spec(LlamaConfig.from_dict(TINY_A)).lm_head_name is None
    assert spec.blocks[2].prefix == "model.layers.2."


def test_to_dict_round_trip():
    for raw in (TINY_A, TINY_B, TINY_C):
        cfg = LlamaConfig.from_dict(raw)
        assert LlamaConfig.from_dict(cfg.to_dict()) == cfg


def test_pages_that_fit_is_the_share_less_everything_else_in_whole_pages():
    from tinyserve_llm_b200.engine.llm import pages_that_fit
    gib = 1 << 30
    # 180 GiB device, 10 GiB in use (weights), 90 % share, 2 GiB step peak, 1 GiB held by graphs, 8 MiB pages
    assert pages_that_fit(180 * gib, 170 * gib, 0.9, 2 * gib, 1 * gib, 8 << 20) == int((162 - 10 - 2 - 1) * 128)
    assert pages_that_fit(180 * gib, 170 * gib, 0.9, 2 * gib, 0, 8 << 20) == pages_that_fit(180 * gib, 170 * gib, 0.9, 2 * gib, 1 * gib, 8 << 20) + 128
    assert pages_that_fit(80 * gib, 8 * gib, 0.9, gib, gib, 8 << 20) < 0          # already over the share: the engine raises
    assert pages_that_fit(gib, gib, 0.5, 0, 0, 3 * (1 << 20)) == 170              # whole pages only


def test_a_head_size_no_kernel_takes_is_refused_when_the_model_is_described():
    """config.json may state any even head_dim; the attention part takes multiples of 16 up to 256 and says so at once."""
    from tiny_configs import TINY_B
    from tinyserve_llm_b200.config.llama import LlamaConfig, llama_model_spec
    from tinyserve_llm_b200.parts.model import declared_tensors
    for bad in (24, 272):
        spec = llama_model_spec(LlamaConfig.from_dict(dict(TINY_B, head_dim=bad)))
        with pytest.raises(ValueError, match=f"head_dim={bad}"):
            declared_tensors(spec)
    declared_tensors(llama_model_spec(LlamaConfig.from_dict(dict(TINY_B, head_dim=48))))
