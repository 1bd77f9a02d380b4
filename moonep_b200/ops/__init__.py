"""Device ops with a tensor-level interface (grouped expert GEMM and companions).
The communication kernels are reached through ``moonep_b200.engine`` / ``Buffer``."""
from . import grouped_gemm

__all__ = ["grouped_gemm"]
