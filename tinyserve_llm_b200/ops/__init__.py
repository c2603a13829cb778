from tinyserve_llm_b200.ops.build import BuildError, build_extension, build_library
from tinyserve_llm_b200.ops.library import KernelError, Ops, get_ops, register_kernel, register_wait_codes

__all__ = ["BuildError", "KernelError", "Ops", "build_extension", "build_library", "get_ops", "register_kernel",
           "register_wait_codes"]
