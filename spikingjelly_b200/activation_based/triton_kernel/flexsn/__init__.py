"""Import path of the reference's ``triton_kernel/flexsn`` (kernels for user-defined neuron dynamics).  The compiler behind
these names is ``spikingjelly_b200.ops.flexsn``: the step function is captured as ATen graphs, emitted as CUDA C++ with the
time loop and every state in registers, compiled by ``nvcc`` and cached.  One compiled object (``FlexSNKernel``) serves what
the reference builds as four Triton kernels (inference, inference with final state only, training forward, backward)."""
from . import custom_ops, hop, info, kernel, template, wrapper  # noqa: F401
from .info import FlexSNInfo, extract_info  # noqa: F401
from .kernel import build_inference_final_state_kernel, build_inference_kernel, build_training_kernels  # noqa: F401
from .wrapper import flexsn_backward, flexsn_forward, flexsn_inference, flexsn_inference_final_state  # noqa: F401
