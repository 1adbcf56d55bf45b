"""Import path of the reference's CuPy back end (``spikingjelly/activation_based/cuda_kernel``).  The kernels themselves are the
ahead-of-time compiled CUDA library of this package (``spikingjelly_b200.ops``); what lives here are the public helpers that user
code imports from this path: spike storage (``tensor_cache``), memory-saving spike layers (``spike_op``), timing / launch
utilities (``cuda_utils``), CUDA C expression builders (``auto_cuda.cfunction``)."""
from . import auto_cuda, cuda_utils, spike_op, tensor_cache  # noqa: F401

__all__ = ["auto_cuda", "cuda_utils", "spike_op", "tensor_cache"]
