from tinyserve_llm_b200.ops.build import BuildError, build_library
from tinyserve_llm_b200.ops.library import KernelError, Ops, get_ops

__all__ = ["BuildError", "KernelError", "Ops", "build_library", "get_ops"]
