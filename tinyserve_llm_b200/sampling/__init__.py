from tinyserve_llm_b200.sampling.sampler import Sampler, draw_key

__all__ = ["Sampler", "draw_key"]
