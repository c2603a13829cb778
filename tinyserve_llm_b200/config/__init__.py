from tinyserve_llm_b200.config.llama import ConfigError, LlamaConfig, llama_model_spec
from tinyserve_llm_b200.config.registry import (
    ARCHITECTURES,
    Architecture,
    load_model_spec,
    read_config_json,
    register_architecture,
    resolve_architecture,
)
from tinyserve_llm_b200.config.spec import (
    AttentionSpec,
    BlockSpec,
    GatedMLPSpec,
    Llama3Scaling,
    ModelSpec,
    PartSpec,
    RMSNormSpec,
    RotarySpec,
    RunEntry,
)

__all__ = [
    "ARCHITECTURES", "Architecture", "AttentionSpec", "BlockSpec", "ConfigError", "GatedMLPSpec",
    "Llama3Scaling", "LlamaConfig", "ModelSpec", "PartSpec", "RMSNormSpec", "RotarySpec", "RunEntry",
    "llama_model_spec", "load_model_spec", "read_config_json", "register_architecture",
    "resolve_architecture",
]
