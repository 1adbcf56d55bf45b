"""FX graph -> kernel source -> loaded module, under the reference's names (``triton_kernel/torch2triton/graph2triton.py:322-470``).
The target language here is CUDA C++: ``generate_triton_code_str(graph, fn_name)`` returns the source of one ``__device__``
function (placeholders become ``float`` parameters, results ``float&`` parameters) and its name; ``compile_triton_code_str``
compiles a complete translation unit with ``nvcc`` for sm_100a into a cached shared object and returns the loaded library, or
the named symbol of it."""
from __future__ import annotations

import hashlib
import re
from typing import Optional, Tuple

import torch
import torch.fx as fx

__all__ = ["generate_triton_code_str", "compile_triton_code_str"]


def generate_triton_code_str(graph: fx.Graph, fn_name: str) -> Tuple[str, str]:
    from ....ops.flexsn import emit_device_function
    gm = graph if isinstance(graph, fx.GraphModule) else fx.GraphModule(torch.nn.Module(), graph)
    stem = re.sub(r"\W", "_", fn_name) or "fn"
    body = emit_device_function(gm, "PLACEHOLDER")
    name = f"{stem}_{hashlib.sha256(body.encode()).hexdigest()[:8]}"
    return body.replace("PLACEHOLDER", name), name


def compile_triton_code_str(triton_code: str, kernel_name: str, name_space: Optional[dict] = None):
    """``triton_code``: a complete ``.cu`` translation unit.  Returns ``getattr(library, kernel_name)`` when the library
    exports that symbol (``extern "C"``), else the library; ``name_space`` receives the library under ``kernel_name``."""
    from ....ops.flexsn import compile_module
    lib = compile_module(triton_code, re.sub(r"\W", "_", kernel_name) or "kernel")
    try:
        obj = getattr(lib, kernel_name)
    except AttributeError:
        obj = lib
    if name_space is not None:
        name_space[kernel_name] = obj
    return obj
