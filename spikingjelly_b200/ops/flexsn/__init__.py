"""Compiler for user-defined neuron dynamics: ATen FX capture -> CUDA C++ -> nvcc -> cached shared object."""
from .codegen import StepGraphs, UnsupportedCore, emit_device_function, emit_module, trace_step, SUPPORTED_OPS
from .compiler import CompileError, cache_dir, compile_module, nvcc_path
from .runtime import (FlexSNKernel, attach_handle_finalizer, build_kernel, flexsn_forward, flexsn_training,
                      lookup_kernel_handle, register_kernel_handle, release_kernel_handle, retain_kernel_handle)
