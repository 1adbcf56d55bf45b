"""FlexSN: a neuron whose dynamics are an arbitrary per-element PyTorch function
``core(*inputs, *states) -> (*outputs, *new_states)``.

With a kernel backend (``"cuda"``; ``"triton"`` and ``"inductor"`` are accepted spellings of it) the step
function is captured as ATen graphs, translated to CUDA C++, compiled by ``nvcc`` for sm_100a on first use and
cached on disk (``spikingjelly_b200.ops.flexsn``).  One kernel runs the whole time loop with the states in
registers; training saves the state after every step and recomputes everything else inside the step.
``"torch"`` runs the Python loop, ``"hop"`` the functional eager scan (same arithmetic, functional
signature).  A core that cannot be compiled — captured tensors, non-elementwise operators, parameters that
need gradients — falls back to the eager scan with a logged warning, as the reference falls back to its HOP
scan (``spikingjelly/activation_based/neuron/flexsn.py:738-1605``).
"""
from __future__ import annotations

import copy
import functools
from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from .. import base
from ...logger import logger

__all__ = ["FlexSN", "FlexSNKernel", "eager_scan"]

_KERNEL_BACKENDS = ("cuda", "triton", "inductor")


def _is_kernel_backend(backend: str) -> bool:
    return backend in _KERNEL_BACKENDS


def _value_requires_grad(value) -> bool:
    if isinstance(value, torch.Tensor):
        return value.requires_grad
    if isinstance(value, nn.Module):
        return any(p.requires_grad for p in value.parameters()) or any(
            _value_requires_grad(v) for k, v in vars(value).items() if not k.startswith("_"))
    if isinstance(value, functools.partial):
        return _core_requires_grad(value)
    if isinstance(value, dict):
        return any(_value_requires_grad(v) for v in value.values())
    if isinstance(value, (tuple, list)):
        return any(_value_requires_grad(v) for v in value)
    return False


def _core_requires_grad(core: Callable) -> bool:
    """True when ``core`` carries tensors that need gradients (module parameters, functor attributes,
    bound-method ``self`` tensors, ``partial`` arguments, closure cells): those gradients only flow
    through the eager paths (``neuron/flexsn.py:359-427``)."""
    if isinstance(core, functools.partial):
        return _core_requires_grad(core.func) or _value_requires_grad(core.args) or _value_requires_grad(core.keywords)
    owner = getattr(core, "__self__", None)
    if owner is not None:
        if _value_requires_grad(owner):
            return True
        d = getattr(owner, "__dict__", None)
        if d is not None and any(_value_requires_grad(v) for v in d.values()):
            return True
    if isinstance(core, nn.Module) and _value_requires_grad(core):
        return True
    if not isinstance(core, nn.Module) and hasattr(core, "__dict__") and not hasattr(core, "__code__"):
        if any(_value_requires_grad(v) for v in vars(core).values()):
            return True
    for cell in getattr(core, "__closure__", None) or ():
        try:
            if _value_requires_grad(cell.cell_contents):
                return True
        except ValueError:
            pass
    return False


def eager_scan(core: Callable, num_inputs: int, num_states: int, num_outputs: int, store_state_seqs: bool,
               *flat_args: torch.Tensor):
    """Functional scan: ``flat_args = (input sequences..., initial states...)`` ->
    ``(output sequences..., state sequences or final states...)``."""
    inputs, states = flat_args[:num_inputs], list(flat_args[num_inputs:])
    T = inputs[0].shape[0]
    outs: List[List[torch.Tensor]] = [[] for _ in range(num_outputs)]
    seqs: List[List[torch.Tensor]] = [[] for _ in range(num_states)]
    for t in range(T):
        res = core(*(x[t] for x in inputs), *states)
        states = list(res[num_outputs:])
        for i in range(num_outputs):
            outs[i].append(res[i])
        if store_state_seqs:
            for j in range(num_states):
                seqs[j].append(states[j])
    out_seqs = [torch.stack(o) for o in outs]
    if store_state_seqs:
        return (*out_seqs, *[torch.stack(s) for s in seqs])
    return (*out_seqs, *states)


class FlexSNKernel:
    """Callable ``(input sequences..., initial states...) -> (output sequences..., state sequences...)``
    around the compiled kernels of one step function, for use outside a module
    (``neuron/flexsn.py:590-736``)."""

    def __init__(self, core: Callable, num_inputs: int, num_states: int, num_outputs: int,
                 example_inputs: Optional[Sequence[torch.Tensor]] = None, requires_grad: Optional[Sequence[bool]] = None):
        from ...ops import flexsn as K
        self._core, self.num_inputs, self.num_states, self.num_outputs = core, num_inputs, num_states, num_outputs
        self._kernel = K.build_kernel(core, num_inputs, num_states, num_outputs, example_inputs, requires_grad)
        self._handle = K.register_kernel_handle(self._kernel)
        self._finalizer = K.attach_handle_finalizer(self, self._handle)

    def __call__(self, *flat_args: torch.Tensor):
        from ...ops import flexsn as K
        if len(flat_args) != self.num_inputs + self.num_states:
            raise ValueError(f"expected {self.num_inputs + self.num_states} tensors, got {len(flat_args)}")
        if torch.is_grad_enabled() and any(a.requires_grad for a in flat_args):
            outs, seqs, _ = K.flexsn_training(self._handle, flat_args)
        else:
            outs, seqs, _ = K.flexsn_forward(self._handle, flat_args, True)
        return (*outs, *seqs)


class FlexSN(base.MemoryModule):
    def __init__(self, core: Callable, num_inputs: int, num_states: int, num_outputs: int,
                 example_inputs: Optional[Tuple[torch.Tensor, ...]] = None,
                 requires_grad: Optional[Tuple[bool, ...]] = None, step_mode: str = "m", backend: str = "triton",
                 store_state_seqs: bool = False, example_outputs: Optional[Tuple[torch.Tensor, ...]] = None):
        super().__init__()
        self.core = core
        self.num_inputs, self.num_states, self.num_outputs = num_inputs, num_states, num_outputs
        if step_mode == "m" and num_inputs == 0:
            raise ValueError("FlexSN step_mode='m' requires at least one input sequence to derive T; got num_inputs=0.")
        if num_inputs + num_states == 0:
            raise ValueError("FlexSN requires at least one input or state tensor.")
        if example_outputs is not None and len(example_outputs) != num_outputs:
            raise ValueError(f"example_outputs must hold {num_outputs} tensors, got {len(example_outputs)}")
        self._output_templates = None if example_outputs is None else [
            (tuple(o.shape), o.dtype) for o in example_outputs]
        self.step_mode = step_mode
        self._kernel = None
        self._handle = None
        self._handle_finalizer = None
        self._build_error: Optional[str] = None
        self._example_inputs, self._requires_grad = example_inputs, requires_grad
        self.backend = backend
        self._store_state_seqs = bool(store_state_seqs)
        self.state_seqs = None
        self.register_memory("states", None)

    # ------------------------------------------------------------------ kernels
    def _build(self) -> None:
        """Trace + generate + compile.  Needs ``nvcc`` but no GPU; failures are recorded, not raised."""
        from ...ops import flexsn as K
        try:
            self._kernel = K.build_kernel(self.core, self.num_inputs, self.num_states, self.num_outputs,
                                          self._example_inputs, self._requires_grad)
            self._handle = K.register_kernel_handle(self._kernel)
            self._handle_finalizer = K.attach_handle_finalizer(self, self._handle)
        except (K.UnsupportedCore, K.CompileError, OSError, RuntimeError, TypeError, ValueError) as e:
            self._kernel, self._handle = None, None
            self._build_error = f"{type(e).__name__}: {e}"
            logger.warning("FlexSN: the step function does not compile (%s); all paths use the eager scan.", self._build_error)

    @property
    def kernel_available(self) -> bool:
        return self._handle is not None

    @property
    def kernel(self):
        return self._kernel_accessor

    def _kernel_accessor(self, *args):
        from ...ops import flexsn as K
        expected = self.num_inputs + self.num_states
        if len(args) != expected:
            raise ValueError(f"FlexSN.kernel expected {expected} tensors ({self.num_inputs} input sequences + "
                             f"{self.num_states} initial states), but got {len(args)}.")
        for i, a in enumerate(args):
            if not isinstance(a, torch.Tensor):
                raise TypeError(f"FlexSN.kernel expected tensor arguments, but arg #{i} is {type(a).__name__}.")
        if self._handle is None or not self._on_one_cuda_device(args):
            raise RuntimeError("FlexSN.kernel is unavailable: the compiled kernels are not ready, or inputs are "
                               "not CUDA tensors on a single device.")
        if torch.is_grad_enabled() and (_core_requires_grad(self.core) or any(a.requires_grad for a in args)):
            outs, seqs, _ = K.flexsn_training(self._handle, args)
        else:
            outs, seqs, _ = K.flexsn_forward(self._handle, args, True)
        return (*outs, *seqs)

    @staticmethod
    def _on_one_cuda_device(tensors) -> bool:
        devs = {t.device for t in tensors}
        return len(devs) == 1 and next(iter(devs)).type == "cuda"

    def __deepcopy__(self, memo):
        # compiled kernels belong to the original's `core`; the copy re-traces its own copy of it
        cls = self.__class__
        new = cls.__new__(cls)
        memo[id(self)] = new
        skip = {"_kernel", "_handle", "_handle_finalizer"}
        for k, v in self.__dict__.items():
            if k not in skip:
                new.__dict__[k] = copy.deepcopy(v, memo)
        new._kernel, new._handle, new._handle_finalizer = None, None, None
        if _is_kernel_backend(new._backend) and self._handle is not None:
            new._build()
        return new

    # ------------------------------------------------------------------ properties
    @property
    def supported_backends(self):
        return ("triton", "torch", "inductor", "hop", "cuda")

    @property
    def backend(self):
        return self._backend

    @backend.setter
    def backend(self, value: str):
        if value not in self.supported_backends:
            raise NotImplementedError(f"{value} is not a supported backend of {self._get_name()}!")
        if _is_kernel_backend(value) and self.step_mode != "m":
            raise RuntimeError(f"Cannot set backend={value!r} when step_mode={self.step_mode!r}; "
                               f"kernel backends require step_mode='m'.")
        self._backend = value
        if _is_kernel_backend(value) and "_kernel" in self.__dict__ and self._handle is None and self._build_error is None:
            self._build()

    @property
    def store_state_seqs(self):
        return self._store_state_seqs

    @store_state_seqs.setter
    def store_state_seqs(self, value: bool):
        self._store_state_seqs = bool(value)
        self.state_seqs = None

    def reset(self):
        super().reset()
        self.state_seqs = None

    @staticmethod
    def init_states(num_states: int, step_mode: str, *args) -> List[torch.Tensor]:
        """Zero states shaped like one step of the first input."""
        if step_mode == "s":
            return [torch.zeros_like(args[0]) for _ in range(num_states)]
        if step_mode == "m":
            if args[0].shape[0] > 0:
                return [torch.zeros_like(args[0][0]) for _ in range(num_states)]
            return [args[0].new_zeros(args[0].shape[1:]) for _ in range(num_states)]
        raise ValueError(f"Unsupported step mode: {step_mode}")

    # ------------------------------------------------------------------ forward
    def single_step_functional_forward(self, inputs, states, **kwargs):
        values = states[0]
        if values is None:
            values = self.init_states(self.num_states, "s", *inputs)
        res = self.core(*inputs, *values)
        return tuple(res[: self.num_outputs]), (list(res[self.num_outputs:]),)

    def _empty_outputs(self, inputs, states):
        if self.num_outputs and self._output_templates is None and self.backend == "torch":
            raise ValueError(f"FlexSN backend='{self.backend}' requires example_outputs for empty multi-step inputs so "
                             "output shapes and dtypes match core's per-step return contract without executing core.")
        x = inputs[0]
        if self._output_templates is None:
            return [x.new_empty((0, *x.shape[1:])) for _ in range(self.num_outputs)]
        return [x.new_empty((0, *shape), dtype=dtype) for shape, dtype in self._output_templates]

    def _multi_step(self, inputs, state_values, store_state_seqs: bool):
        from ...ops import flexsn as K
        if self.backend not in self.supported_backends:
            raise ValueError(f"Unsupported backend: {self.backend}")
        if state_values is None:
            state_values = self.init_states(self.num_states, "m", *inputs)
        state_values = list(state_values)
        T = inputs[0].shape[0]
        if T == 0:
            outs = self._empty_outputs(inputs, state_values)
            seqs = [s.new_empty((0, *s.shape)) for s in state_values] if store_state_seqs else None
            return tuple(outs), ((seqs, state_values) if store_state_seqs else (state_values,))

        flat = [*inputs, *state_values]
        if _is_kernel_backend(self.backend) and self._handle is not None and self._on_one_cuda_device(flat):
            core_grad = _core_requires_grad(self.core)
            no_grad = not torch.is_grad_enabled() or (not any(t.requires_grad for t in flat) and not core_grad)
            if no_grad:
                outs, seqs, last = K.flexsn_forward(self._handle, flat, store_state_seqs)
                return tuple(outs), ((list(seqs), list(last)) if store_state_seqs else (list(last),))
            if not core_grad and self._kernel.has_backward:
                outs, seqs, last = K.flexsn_training(self._handle, flat)
                return tuple(outs), ((seqs, last) if store_state_seqs else (last,))

        res = eager_scan(self.core, self.num_inputs, self.num_states, self.num_outputs, store_state_seqs, *flat)
        outs, rest = res[: self.num_outputs], list(res[self.num_outputs:])
        if store_state_seqs:
            last = [seq[-1] for seq in rest]
            return tuple(outs), (rest, last)
        return tuple(outs), (rest,)

    def multi_step_functional_forward(self, inputs, states, **kwargs):
        return self._multi_step(inputs, states[0], False)

    def single_step_forward(self, *args: torch.Tensor):
        outs, (self._memories["states"],) = self.single_step_functional_forward(args, (self._memories["states"],))
        return tuple(outs)

    def multi_step_forward(self, *args: torch.Tensor):
        outs, updated = self._multi_step(tuple(args), self._memories["states"], self.store_state_seqs)
        if self.store_state_seqs:
            self.state_seqs, self._memories["states"] = updated
        else:
            (self._memories["states"],) = updated
        return list(outs)

    def forward(self, *args: torch.Tensor):
        if self.step_mode == "s":
            outs = self.single_step_forward(*args)
        elif self.step_mode == "m":
            outs = self.multi_step_forward(*args)
        else:
            raise ValueError(self.step_mode)
        return outs[0] if len(outs) == 1 else outs

    def extra_repr(self):
        name = getattr(self.core, "__name__", type(self.core).__name__)
        if isinstance(self.core, functools.partial):
            name = f"partial({getattr(self.core.func, '__name__', type(self.core.func).__name__)})"
        return (f"core={name}, num_inputs={self.num_inputs}, num_states={self.num_states}, "
                f"num_outputs={self.num_outputs}, step_mode={self.step_mode!r}, backend={self.backend!r}")
