"""Single-step kernels assembled from code fragments (``cuda_kernel/neuron_kernel/single_step/base.py`` of the reference): element-wise
over ``numel`` values, ``(x, v) -> (spike, v_next, h)`` forward and ``(grad_spike, grad_v_next, h) -> (grad_x, grad_v)`` backward.
``dtype`` is ``"float"``."""
from __future__ import annotations

from pathlib import Path
from typing import Callable

from ...auto_cuda import base as auto_cuda_base

__all__ = ["NeuronFPKernel", "NeuronBPKernel"]


def _only_float(dtype: str) -> None:
    if dtype != "float":
        raise NotImplementedError(f"fragment-assembled neuron kernels are written for dtype 'float', got {dtype!r}")


class NeuronFPKernel(auto_cuda_base.CKernel1D):
    def __init__(self, hard_reset: bool, dtype: str):
        _only_float(dtype)
        super().__init__(kernel_name=f"{type(self).__name__}_{dtype}_{'hard_reset' if hard_reset else 'soft_reset'}")
        self.hard_reset, self.dtype = hard_reset, dtype
        self.add_param(ctype=f"const {dtype} *", cname="x")
        self.add_param(ctype=f"const {dtype} *", cname="v")
        self.add_param(ctype=f"{dtype} *", cname="h")
        self.add_param(ctype=f"{dtype} *", cname="spike")
        self.add_param(ctype=f"{dtype} *", cname="v_next")
        self.add_param(ctype=f"{dtype} &", cname="v_th")
        if hard_reset:
            self.add_param(ctype=f"{dtype} &", cname="v_reset")

    def neuronal_charge(self) -> str:
        """Statements writing ``h[index]`` from ``x[index]`` and ``v[index]``."""
        return "// neuronal_charge should be defined here!"

    @property
    def core(self) -> str:
        reset = ("v_next[index] = spike[index] * v_reset + (1.0f - spike[index]) * h[index];" if self.hard_reset
                 else "v_next[index] = h[index] - spike[index] * v_th;")
        return "\n".join("        " + s for s in (*self.neuronal_charge().strip().splitlines(),
                                                  "spike[index] = (h[index] - v_th >= 0.0f) ? 1.0f : 0.0f;", reset))

    @core.setter
    def core(self, value) -> None:
        pass


class NeuronBPKernel(auto_cuda_base.CKernel1D):
    def __init__(self, surrogate_function: Callable, hard_reset: bool, detach_reset: bool, dtype: str):
        _only_float(dtype)
        super().__init__(kernel_name=f"{type(self).__name__}_{dtype}_{'hard_reset' if hard_reset else 'soft_reset'}_"
                                     f"{'detach_reset' if detach_reset else 'nodetach_reset'}")
        self.surrogate_function, self.hard_reset, self.detach_reset, self.dtype = surrogate_function, hard_reset, detach_reset, dtype
        self.add_param(ctype=f"const {dtype} *", cname="grad_spike")
        self.add_param(ctype=f"const {dtype} *", cname="grad_v_next")
        self.add_param(ctype=f"const {dtype} *", cname="h")
        self.add_param(ctype=f"{dtype} *", cname="grad_x")
        self.add_param(ctype=f"{dtype} *", cname="grad_v")
        self.add_param(ctype=f"{dtype} &", cname="v_th")
        if hard_reset:
            self.add_param(ctype=f"{dtype} &", cname="v_reset")
        from .....ops import __file__ as ops_file
        self.extra_headers = (Path(ops_file).parent / "csrc" / "surrogate.cuh").read_text()

    def grad_h_to_v(self) -> str:
        """Statement defining ``const float grad_h_to_v`` = d h / d v."""
        return "// grad_h_to_v should be defined here!"

    def grad_h_to_x(self) -> str:
        """Statement defining ``const float grad_h_to_x`` = d h / d x."""
        return "// grad_h_to_x should be defined here!"

    @property
    def core(self) -> str:
        sg = self.surrogate_function.cuda_codes(y="grad_s_to_h", x="over_th", dtype="float")
        if self.hard_reset:
            v_to_h = ("const float grad_v_to_h = 1.0f - spike_now;" if self.detach_reset
                      else "const float grad_v_to_h = 1.0f - spike_now + (v_reset - h[index]) * grad_s_to_h;")
        else:
            v_to_h = "const float grad_v_to_h = 1.0f;" if self.detach_reset else "const float grad_v_to_h = 1.0f - v_th * grad_s_to_h;"
        lines = ["const float over_th = h[index] - v_th;", "const float spike_now = (over_th >= 0.0f) ? 1.0f : 0.0f;", sg, v_to_h,
                 "const float grad_h = grad_spike[index] * grad_s_to_h + grad_v_next[index] * grad_v_to_h;",
                 *self.grad_h_to_v().strip().splitlines(), *self.grad_h_to_x().strip().splitlines(),
                 "grad_x[index] = grad_h * grad_h_to_x;", "grad_v[index] = grad_h * grad_h_to_v;"]
        return "\n".join("        " + s for s in lines)

    @core.setter
    def core(self, value) -> None:
        pass
