"""
Typed configuration of the Llama dense decoder, read from the keys of its own config.json.

Reference behaviour this mirrors: rope settings under `rope_parameters` or at the top level
(model/llama.py:86-104), head_dim defaulting to hidden_size // num_attention_heads (:197),
attention_bias / mlp_bias must be false (:193, :232), hidden_act must be "silu" (:219),
tie_word_embeddings defaulting to False (:294), eos_token_id an int or a list whose first element
counts (engine/llm_engine.py:105-110).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from tinyserve_llm_b200.config.spec import (
    AttentionSpec,
    BlockSpec,
    GatedMLPSpec,
    Llama3Scaling,
    ModelSpec,
    RMSNormSpec,
    RotarySpec,
    RunEntry,
)


class ConfigError(ValueError):
    """config.json is missing a key, or asks for something this engine does not implement."""


_REQUIRED = (
    "vocab_size",
    "hidden_size",
    "intermediate_size",
    "num_hidden_layers",
    "num_attention_heads",
    "rms_norm_eps",
    "max_position_embeddings",
)


def _positive_int(raw: Mapping[str, Any], key: str) -> int:
    value = raw[key]
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ConfigError(f"config.json: {key} must be a positive integer, got {value!r}")
    return value


@dataclass(frozen=True)
class LlamaConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    hidden_act: str
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: Llama3Scaling | None
    max_position_embeddings: int
    tie_word_embeddings: bool
    eos_token_id: int                # -1: none

    architecture = "LlamaForCausalLM"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "LlamaConfig":
        missing = [k for k in _REQUIRED if k not in raw]
        if missing:
            raise ConfigError(f"config.json lacks required keys: {missing}")
        hidden = _positive_int(raw, "hidden_size")
        heads = _positive_int(raw, "num_attention_heads")
        kv_heads = raw.get("num_key_value_heads")
        if kv_heads is None:
            kv_heads = heads
        if not isinstance(kv_heads, int) or kv_heads <= 0 or heads % kv_heads:
            raise ConfigError(
                f"config.json: num_key_value_heads={kv_heads!r} must divide num_attention_heads={heads}")
        head_dim = raw.get("head_dim") or hidden // heads
        if not isinstance(head_dim, int) or head_dim <= 0 or head_dim % 2:
            raise ConfigError(f"config.json: head_dim={head_dim!r} must be a positive even integer")
        if raw.get("attention_bias", False):
            raise ConfigError("config.json: attention_bias=true is not supported")
        if raw.get("mlp_bias", False):
            raise ConfigError("config.json: mlp_bias=true is not supported")
        act = raw.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act={act!r} is not supported; have ['silu']")
        theta, scaling = _rope_settings(raw, _positive_int(raw, "max_position_embeddings"))
        eos = raw.get("eos_token_id")
        if isinstance(eos, list):
            eos = eos[0] if eos else None
        eps = raw["rms_norm_eps"]
        if not isinstance(eps, (int, float)) or isinstance(eps, bool) or not eps > 0:
            raise ConfigError(f"config.json: rms_norm_eps must be a positive number, got {eps!r}")
        return cls(
            vocab_size=_positive_int(raw, "vocab_size"),
            hidden_size=hidden,
            intermediate_size=_positive_int(raw, "intermediate_size"),
            num_hidden_layers=_positive_int(raw, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            hidden_act=act,
            rms_norm_eps=float(eps),
            rope_theta=theta,
            rope_scaling=scaling,
            max_position_embeddings=_positive_int(raw, "max_position_embeddings"),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            eos_token_id=-1 if eos is None else int(eos),
        )

    def to_dict(self) -> dict[str, Any]:
        """The config.json this configuration is read back from (hub spelling)."""
        out: dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "hidden_act": self.hidden_act,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": None,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": False,
            "mlp_bias": False,
            "eos_token_id": None if self.eos_token_id < 0 else self.eos_token_id,
            "torch_dtype": "bfloat16",
        }
        if self.rope_scaling is not None:
            s = self.rope_scaling
            out["rope_scaling"] = {
                "rope_type": "llama3",
                "factor": s.factor,
                "low_freq_factor": s.low_freq_factor,
                "high_freq_factor": s.high_freq_factor,
                "original_max_position_embeddings": s.original_max_position_embeddings,
            }
        return out


def _rope_settings(raw: Mapping[str, Any], max_positions: int) -> tuple[float, Llama3Scaling | None]:
    params = raw.get("rope_parameters")
    if params:
        theta = params.get("rope_theta", raw.get("rope_theta", 10000.0))
        scaling = params
    else:
        theta = raw.get("rope_theta", 10000.0)
        scaling = raw.get("rope_scaling")
    if not isinstance(theta, (int, float)) or isinstance(theta, bool) or not theta > 0:
        raise ConfigError(f"config.json: rope_theta must be a positive number, got {theta!r}")
    if scaling is None:
        return float(theta), None
    rope_type = scaling.get("rope_type", scaling.get("type", "default"))
    if rope_type == "default":
        return float(theta), None
    if rope_type != "llama3":
        raise ConfigError(f"config.json: rope_type {rope_type!r} is not supported; have ['default', 'llama3']")
    try:
        return float(theta), Llama3Scaling(
            factor=float(scaling["factor"]),
            low_freq_factor=float(scaling["low_freq_factor"]),
            high_freq_factor=float(scaling["high_freq_factor"]),
            original_max_position_embeddings=int(
                scaling.get("original_max_position_embeddings", max_positions)),
        )
    except KeyError as exc:
        raise ConfigError(f"config.json: llama3 rope scaling lacks {exc.args[0]!r}") from None


def llama_model_spec(config: LlamaConfig) -> ModelSpec:
    """Every Llama layer is the same pre-norm block; each runs once, in order, with its own cache entry."""
    rotary = RotarySpec(
        head_dim=config.head_dim,
        theta=config.rope_theta,
        max_positions=config.max_position_embeddings,
        scaling=config.rope_scaling,
    )
    attention = AttentionSpec(
        hidden_size=config.hidden_size,
        num_heads=config.num_attention_heads,
        num_kv_heads=config.num_key_value_heads,
        head_dim=config.head_dim,
        scale=config.head_dim ** -0.5,
        window=0,
        position=rotary,
    )
    mlp = GatedMLPSpec(
        hidden_size=config.hidden_size,
        intermediate_size=config.intermediate_size,
        activation=config.hidden_act,
    )
    norm = RMSNormSpec(size=config.hidden_size, eps=config.rms_norm_eps)
    blocks = tuple(
        BlockSpec(
            arrangement="pre_norm",
            mixer=attention,
            feed_forward=mlp,
            mixer_norm=norm,
            feed_forward_norm=norm,
            prefix=f"model.layers.{i}.",
        )
        for i in range(config.num_hidden_layers)
    )
    return ModelSpec(
        architecture=config.architecture,
        vocab_size=config.vocab_size,
        hidden_size=config.hidden_size,
        blocks=blocks,
        run=tuple(RunEntry(block=i, cache_entry=i) for i in range(config.num_hidden_layers)),
        final_norm=norm,
        embedding_name="model.embed_tokens.weight",
        final_norm_prefix="model.norm.",
        lm_head_name=None if config.tie_word_embeddings else "lm_head.weight",
        max_positions=config.max_position_embeddings,
        eos_token_id=config.eos_token_id,
        # model/loader.py:19, 43-47 of the reference: a tied checkpoint may still carry lm_head.weight, and
        # checkpoints of older exporters carry each layer's rotary inv_freq buffer
        optional_tensors=("lm_head.weight",) if config.tie_word_embeddings else (),
        ignored_suffixes=("rotary_emb.inv_freq",),
    )
