"""Import path of the reference's Triton back end (``spikingjelly/activation_based/triton_kernel``).  This package has no Triton
code: the neuron kernels are the native CUDA scan kernels (``backend="triton"`` selects them), custom neurons are compiled by
``ops.flexsn``.  The helpers user code imports from this path are kept: spike bit compression and the fp8 capability probe."""
from . import compress, fp8_capability  # noqa: F401
from .compress import bit_spike_compress, bit_spike_decompress  # noqa: F401

__all__ = ["compress", "fp8_capability", "bit_spike_compress", "bit_spike_decompress"]
