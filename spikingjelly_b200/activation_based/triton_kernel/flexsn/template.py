"""Kernel source by direction (``triton_kernel/flexsn/template.py`` of the reference fills Triton templates with the core's
code string; here the generator emits one CUDA translation unit per step function, and these functions return it).  The first
argument is the traced step function (``ops.flexsn.StepGraphs``, e.g. ``kernel.graphs``); ``core_name`` and ``info`` are
accepted for call compatibility.  Returns ``(source, entry point)``: ``flexsn_forward`` / ``flexsn_backward`` are the
``extern "C"`` launchers of the translation unit."""
from __future__ import annotations

__all__ = ["get_flexsn_inference_kernel", "get_flexsn_inference_final_state_kernel", "get_flexsn_forward_kernel",
           "get_flexsn_backward_kernel"]


def _source(graphs):
    from ....ops.flexsn import StepGraphs, emit_module
    if not isinstance(graphs, StepGraphs):
        raise TypeError("expected the traced step function (ops.flexsn.StepGraphs); the CUDA generator works from graphs, not "
                        "from a code string")
    return emit_module(graphs)


def get_flexsn_inference_kernel(graphs, core_name: str = "core", info=None):
    return _source(graphs), "flexsn_forward"


get_flexsn_inference_final_state_kernel = get_flexsn_forward_kernel = get_flexsn_inference_kernel


def get_flexsn_backward_kernel(graphs, core_name: str = "core", info=None):
    if graphs.joint is None:
        raise ValueError("the step function was traced without a backward graph")
    return _source(graphs), "flexsn_backward"
