"""Forward-through-time and backward-through-time kernels assembled from code fragments, and the glue that runs them inside
``torch.autograd.Function`` (``cuda_kernel/neuron_kernel/multi_step/base.py:30-700`` of the reference).

A forward kernel walks ``t`` upwards over ``[T, N]`` tensors: charge ``h_seq[t]`` from ``x_seq[t]`` and ``v_v_seq[t]`` (the fragment
:meth:`NeuronFPTTKernel.neuronal_charge`), fire, reset into ``v_v_seq[t + dt]`` (``v_v_seq`` holds ``T + 1`` rows: the initial
potential, then every step's).  A backward kernel walks downwards with the running ``grad_h``:

    grad_h = grad_spike_seq[t] * sg'(h - v_th) + (grad_v_seq[t] + grad_h * grad_h_next_to_v) * grad_v_to_h
    grad_x_seq[t] = grad_h * grad_h_to_x

where the fragments :meth:`NeuronBPTTKernel.grad_h_next_to_v` and :meth:`grad_h_to_x` define ``const float grad_h_next_to_v``
and ``const float grad_h_to_x``.  ``dtype`` is ``"float"``."""
from __future__ import annotations

from pathlib import Path
from typing import Callable, Iterable

import torch

from ..... import configure
from ...auto_cuda import base as auto_cuda_base

__all__ = ["NeuronFPTTKernel", "NeuronBPTTKernel", "if_requires_grad", "prepare_forward_meta", "new_tensors", "NeuronATGFBase"]


def _only_float(dtype: str) -> None:
    if dtype != "float":
        raise NotImplementedError(f"fragment-assembled neuron kernels are written for dtype 'float', got {dtype!r}; 16-bit tensors run "
                                  "through the native scan kernels (the functional entry points of this package)")


def _reset_name(hard: bool) -> str:
    return "hard_reset" if hard else "soft_reset"


class NeuronFPTTKernel(auto_cuda_base.CKernel2D):
    def __init__(self, hard_reset: bool, dtype: str):
        _only_float(dtype)
        super().__init__(kernel_name=f"{type(self).__name__}_{dtype}_{_reset_name(hard_reset)}", reverse=False)
        self.hard_reset, self.dtype = hard_reset, dtype
        self.add_param(ctype=f"const {dtype} *", cname="x_seq")
        self.add_param(ctype=f"{dtype} *", cname="v_v_seq")
        self.add_param(ctype=f"{dtype} *", cname="h_seq")
        self.add_param(ctype=f"{dtype} *", cname="spike_seq")
        self.add_param(ctype=f"{dtype} &", cname="v_th")
        if hard_reset:
            self.add_param(ctype=f"{dtype} &", cname="v_reset")

    def neuronal_charge(self) -> str:
        """CUDA statements that write ``h_seq[t]`` from ``x_seq[t]`` and ``v_v_seq[t]`` (plus any parameter the subclass added),
        e.g. ``h_seq[t] = x_seq[t] + v_v_seq[t];`` for the IF neuron."""
        return "// neuronal_charge should be defined here!"

    @property
    def core(self) -> str:
        reset = ("v_v_seq[t + dt] = spike_seq[t] * v_reset + (1.0f - spike_seq[t]) * h_seq[t];" if self.hard_reset
                 else "v_v_seq[t + dt] = h_seq[t] - spike_seq[t] * v_th;")
        return "\n".join("          " + line for line in (*self.neuronal_charge().strip().splitlines(),
                                                          "spike_seq[t] = (h_seq[t] - v_th >= 0.0f) ? 1.0f : 0.0f;", reset))

    @core.setter
    def core(self, value) -> None:        # the base class assigns "" in its constructor
        pass


class NeuronBPTTKernel(auto_cuda_base.CKernel2D):
    def __init__(self, surrogate_function: Callable, hard_reset: bool, detach_reset: bool, dtype: str):
        _only_float(dtype)
        super().__init__(kernel_name=f"{type(self).__name__}_{dtype}_{_reset_name(hard_reset)}_"
                                     f"{'detach_reset' if detach_reset else 'nodetach_reset'}", reverse=True)
        self.surrogate_function, self.hard_reset, self.detach_reset, self.dtype = surrogate_function, hard_reset, detach_reset, dtype
        self.add_param(ctype=f"const {dtype} *", cname="grad_spike_seq")
        self.add_param(ctype=f"const {dtype} *", cname="grad_v_seq")
        self.add_param(ctype=f"const {dtype} *", cname="h_seq")
        self.add_param(ctype=f"{dtype} *", cname="grad_x_seq")
        self.add_param(ctype=f"{dtype} *", cname="grad_v_init")
        self.add_param(ctype=f"{dtype} &", cname="v_th")
        if hard_reset:
            self.add_param(ctype=f"{dtype} &", cname="v_reset")
        from .....ops import __file__ as ops_file          # device function sjb200::surrogate_grad<ID>(x, p0, p1)
        self.extra_headers = (Path(ops_file).parent / "csrc" / "surrogate.cuh").read_text()

    def grad_h_next_to_v(self) -> str:
        """Statement defining ``const float grad_h_next_to_v`` = d h[t+1] / d v[t], e.g. ``= 1.0f`` for the IF neuron."""
        return "// grad_h_next_to_v should be defined here!"

    def grad_h_to_x(self) -> str:
        """Statement defining ``const float grad_h_to_x`` = d h[t] / d x[t]."""
        return "// grad_h_to_x should be defined here!"

    @property
    def pre_core(self) -> str:
        return "          float grad_h = 0.0f;\n" + self._extra_pre_core()

    @pre_core.setter
    def pre_core(self, value) -> None:
        pass

    def _extra_pre_core(self) -> str:
        return ""

    @property
    def post_core(self) -> str:
        return ("          {\n            " + self.grad_h_next_to_v().strip() + "\n            grad_v_init[index] = grad_h * grad_h_next_to_v;\n          }\n"
                + self._extra_post_core())

    @post_core.setter
    def post_core(self, value) -> None:
        pass

    def _extra_post_core(self) -> str:
        return ""

    def _extra_core(self) -> str:
        """Statements placed after ``grad_h`` of this step is known (e.g. a parameter gradient)."""
        return ""

    @property
    def core(self) -> str:
        sg = self.surrogate_function.cuda_codes(y="grad_s_to_h", x="over_th", dtype="float")
        if self.hard_reset:
            v_to_h = ("const float grad_v_to_h = 1.0f - spike;" if self.detach_reset
                      else "const float grad_v_to_h = 1.0f - spike + (v_reset - h_seq[t]) * grad_s_to_h;")
        else:
            v_to_h = "const float grad_v_to_h = 1.0f;" if self.detach_reset else "const float grad_v_to_h = 1.0f - v_th * grad_s_to_h;"
        lines = ["const float over_th = h_seq[t] - v_th;", "const float spike = (over_th >= 0.0f) ? 1.0f : 0.0f;", sg, v_to_h,
                 *self.grad_h_next_to_v().strip().splitlines(),
                 "grad_h = grad_spike_seq[t] * grad_s_to_h + (grad_v_seq[t] + grad_h * grad_h_next_to_v) * grad_v_to_h;",
                 *self.grad_h_to_x().strip().splitlines(), "grad_x_seq[t] = grad_h * grad_h_to_x;", *self._extra_core().strip().splitlines()]
        return "\n".join("          " + line for line in lines if line)

    @core.setter
    def core(self, value) -> None:
        pass


def if_requires_grad(items: Iterable) -> bool:
    return any(isinstance(i, torch.Tensor) and i.requires_grad for i in items)


def _blocks(n: int) -> int:
    return (n + configure.cuda_threads - 1) // configure.cuda_threads


def prepare_forward_meta(py_dict: dict, ref: str = "x_seq"):
    """Adds ``numel`` and ``N`` of the ``[T, N]`` tensor ``py_dict[ref]``; returns ``(blocks, threads, py_dict)``."""
    t = py_dict[ref]
    py_dict["numel"], py_dict["N"] = t.numel(), t.shape[1]
    return _blocks(t.shape[1]), configure.cuda_threads, py_dict


def new_tensors(news: tuple, py_dict: dict, ref: str = "x_seq") -> None:
    """Zero tensors shaped like ``py_dict[ref]`` under each name of ``news``, carved from one allocation."""
    t = py_dict[ref]
    block = torch.zeros((len(news) * t.shape[0], *t.shape[1:]), device=t.device, dtype=t.dtype)
    for name, part in zip(news, block.split(t.shape[0])):
        py_dict[name] = part


class NeuronATGFBase:
    """Helpers for the ``forward`` / ``backward`` of an autograd function around a kernel pair."""

    @staticmethod
    def pre_forward(py_dict: dict):
        """``py_dict`` holds at least ``x_seq [T, N]``, ``v_init [N]``, ``v_th`` and ``v_reset`` (``None`` = soft reset, the key is then
        dropped).  Adds ``h_seq``, ``spike_seq``, ``v_v_seq`` (``v_init`` followed by room for T steps), ``numel``, ``N``.
        Returns ``(requires_grad, blocks, threads, py_dict)``."""
        requires_grad = if_requires_grad(py_dict.values())
        if py_dict.get("v_reset", None) is None:
            py_dict.pop("v_reset", None)
        new_tensors(("h_seq", "spike_seq", "v_seq"), py_dict)
        py_dict["v_v_seq"] = torch.cat((py_dict.pop("v_init").detach().unsqueeze(0), py_dict.pop("v_seq")))
        blocks, threads, py_dict = prepare_forward_meta(py_dict)
        return requires_grad, blocks, threads, py_dict

    @staticmethod
    def ctx_save(ctx, requires_grad: bool, *args, **kwargs) -> None:
        if requires_grad:
            ctx.save_for_backward(*args)
            for k, v in kwargs.items():
                setattr(ctx, k, v)

    @staticmethod
    def pre_backward(ctx, grad_spike_seq: torch.Tensor, grad_v_seq: torch.Tensor):
        """``(backward_kernel, blocks, threads, py_dict)`` with zeroed ``grad_x_seq`` / ``grad_v_init`` in ``py_dict``."""
        block = torch.zeros((grad_spike_seq.shape[0] + 1, *grad_spike_seq.shape[1:]), device=grad_spike_seq.device, dtype=grad_spike_seq.dtype)
        py_dict = {"numel": ctx.numel, "N": ctx.N, "grad_spike_seq": grad_spike_seq, "grad_v_seq": grad_v_seq, "h_seq": ctx.saved_tensors[0],
                   "grad_x_seq": block[:-1], "grad_v_init": block[-1], "v_th": ctx.v_th}
        if ctx.v_reset is not None:
            py_dict["v_reset"] = ctx.v_reset
        return ctx.backward_kernel, ctx.blocks, ctx.threads, py_dict
