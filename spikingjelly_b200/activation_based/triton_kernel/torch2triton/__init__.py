"""Import path of the reference's ``triton_kernel/torch2triton`` (PyTorch function -> FX graph -> kernel source).  The same two
stages exist here with CUDA C++ as the target: ``torch2graph`` captures ATen graphs, ``graph2triton`` turns a graph into a
``__device__`` function and compiles complete translation units (``ops/flexsn/codegen.py``, ``compiler.py``)."""
from . import graph2triton, torch2graph  # noqa: F401
from .graph2triton import compile_triton_code_str, generate_triton_code_str  # noqa: F401
from .torch2graph import generate_forward_and_backward_graph, generate_inference_graph  # noqa: F401
