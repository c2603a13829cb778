from tinyserve_llm_b200.weights.loader import CheckpointError, checkpoint_files, load_tensors
from tinyserve_llm_b200.weights.random_init import random_tensors, write_random_model
from tinyserve_llm_b200.weights.safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors

__all__ = ["CheckpointError", "SafetensorsError", "SafetensorsFile", "checkpoint_files", "load_tensors",
           "random_tensors", "write_random_model", "write_safetensors"]
