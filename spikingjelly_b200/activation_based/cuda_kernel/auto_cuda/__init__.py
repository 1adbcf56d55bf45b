"""String builders for element-wise CUDA C expressions (``cuda_kernel/auto_cuda`` of the reference, where they feed the CuPy
source generator).  Here they serve user code that assembles ``cuda_codes`` of a custom surrogate or neuron by hand; kernels
for custom neurons are normally produced by the FlexSN compiler (``ops/flexsn``), which needs none of this."""
from . import cfunction  # noqa: F401

__all__ = ["cfunction"]
