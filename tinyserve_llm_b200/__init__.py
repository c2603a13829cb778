"""
tinyserve_llm_b200: a single-GPU inference engine for NVIDIA B200 (sm_100a) with the capabilities
tejkas/tinyserve-llm shows for the Llama dense decoder: typed configuration and registry, named
safetensors weights, layers put together from parts, a paged cache manager with prefix reuse, one
step function, a cache-aware scheduler with prompt portions, sampling, and a trace replay program.
"""

from tinyserve_llm_b200.engine.llm import LLM, CacheConfig, Completion, StepRecord
from tinyserve_llm_b200.engine.scheduler import SchedulerConfig
from tinyserve_llm_b200.engine.sequence import SamplingParams

__all__ = ["LLM", "CacheConfig", "Completion", "SamplingParams", "SchedulerConfig", "StepRecord"]
