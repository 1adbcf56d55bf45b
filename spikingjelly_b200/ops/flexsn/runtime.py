"""Launch side of the generated neuron kernels: argument packing, the integer handle registry that lets
compiled kernels travel through ``torch.library`` operator schemas, the operators themselves
(``sjb200_flexsn::forward`` / ``::backward`` with fake implementations) and the autograd wrapper.

Role of ``triton_kernel/flexsn/wrapper.py:26-…`` and ``flexsn/custom_ops.py:89-1118`` in the reference.
"""
from __future__ import annotations

import contextlib
import ctypes
import threading
import weakref
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from . import codegen, compiler

__all__ = ["FlexSNKernel", "build_kernel", "register_kernel_handle", "retain_kernel_handle", "release_kernel_handle",
           "lookup_kernel_handle", "attach_handle_finalizer", "flexsn_forward", "flexsn_training"]

_DTYPE_CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def _struct(name: str, fields: Sequence[Tuple[str, int]]):
    spec = [(f, ctypes.c_void_p * n) for f, n in fields] + [("n", ctypes.c_longlong), ("T", ctypes.c_int)]
    return type(name, (ctypes.Structure,), {"_fields_": spec})


def _on_device(device: torch.device):
    """A device guard that costs nothing when ``device`` is already current (the usual case: one process per GPU)."""
    if device.index is None or device.index == torch.cuda.current_device():
        return contextlib.nullcontext()
    return torch.cuda.device(device)


def _forward_flat(handle: int, flat_args: Sequence[torch.Tensor], store_state_seqs: bool) -> List[torch.Tensor]:
    """Eager calls go straight to the kernel; the registered operator (Python dispatch, ~100 us per call) is only
    needed when a tracer has to see one opaque node."""
    if torch.compiler.is_compiling():
        return torch.ops.sjb200_flexsn.forward(handle, list(flat_args), store_state_seqs)
    k = lookup_kernel_handle(handle)
    outs, seqs, last = k.forward(flat_args[:k.NI], flat_args[k.NI:], store_state_seqs)
    return [*outs, *(seqs or []), *last]


class FlexSNKernel:
    """One compiled step function.  ``forward`` and ``backward`` launch on the current stream of the
    tensors' device and never synchronise."""

    def __init__(self, graphs: codegen.StepGraphs, lib: ctypes.CDLL):
        self.graphs = graphs
        self.lib = lib
        NI, NS, NO = graphs.num_inputs, graphs.num_states, graphs.num_outputs
        nsd, nod = max(NS, 1), max(NO, 1)
        self.NI, self.NS, self.NO = NI, NS, NO
        self._Fwd = _struct("FwdArgs", [("inp", NI), ("s0", nsd), ("out", nod), ("s_seq", nsd), ("s_last", nsd)])
        self._Bwd = _struct("BwdArgs", [("inp", NI), ("s0", nsd), ("s_seq", nsd), ("g_out", nod), ("g_seq", nsd),
                                        ("g_last", nsd), ("g_in", NI), ("g_s0", nsd)])
        lib.flexsn_forward.restype = ctypes.c_int
        lib.flexsn_forward.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        self.has_backward = graphs.joint is not None
        if self.has_backward:
            lib.flexsn_backward.restype = ctypes.c_int
            lib.flexsn_backward.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]

    # ------------------------------------------------------------------ checks
    def _check(self, inputs: Sequence[torch.Tensor], states: Sequence[torch.Tensor]):
        x0 = inputs[0]
        if x0.dtype not in _DTYPE_CODE:
            raise TypeError(f"compiled neuron kernels run on float32/float16/bfloat16, got {x0.dtype}")
        for x in inputs:
            if x.shape != x0.shape or x.dtype != x0.dtype or x.device != x0.device:
                raise ValueError("all input sequences must share shape, dtype and device")
        for s in states:
            if s.shape != x0.shape[1:] or s.dtype != x0.dtype or s.device != x0.device:
                raise ValueError("every state must have the shape of one step of the input, its dtype and device")
        T = x0.shape[0]
        n = x0[0].numel() if T > 0 else int(torch.Size(x0.shape[1:]).numel())
        return T, n, _DTYPE_CODE[x0.dtype]

    @staticmethod
    def _vec(tensors: Sequence[Optional[torch.Tensor]], n: int, itemsize: int) -> int:
        """1 when the launch may use four-element accesses (16 bytes in fp32, 8 in 16-bit types), else 0."""
        if n % 4:
            return 0
        return int(all(t is None or t.data_ptr() % 16 == 0 for t in tensors))

    @staticmethod
    def _fill(arr, tensors: Sequence[Optional[torch.Tensor]]):
        for i, t in enumerate(tensors):
            arr[i] = None if t is None else t.data_ptr()

    # ------------------------------------------------------------------ launches
    def forward(self, inputs: Sequence[torch.Tensor], states: Sequence[torch.Tensor], store_state_seqs: bool):
        """-> (output sequences, state sequences or None, final states)."""
        from .. import counters
        inputs = [x.contiguous() for x in inputs]
        states = [s.contiguous() for s in states]
        T, n, code = self._check(inputs, states)
        x0 = inputs[0]
        outs = [torch.empty_like(x0) for _ in range(self.NO)]
        seqs = [torch.empty_like(x0) for _ in range(self.NS)] if store_state_seqs else None
        last = [torch.empty_like(s) for s in states]
        if T == 0 or n == 0:
            for l, s in zip(last, states):
                l.copy_(s)
            return outs, seqs, last
        a = self._Fwd()
        self._fill(a.inp, inputs)
        self._fill(a.s0, states)
        self._fill(a.out, outs)
        self._fill(a.s_seq, seqs if seqs is not None else [None] * self.NS)
        self._fill(a.s_last, last)
        a.n, a.T = n, T
        vec = self._vec([*inputs, *states, *outs, *(seqs or []), *last], n, x0.element_size())
        with _on_device(x0.device):
            stream = torch.cuda.current_stream(x0.device).cuda_stream
            rc = self.lib.flexsn_forward(ctypes.byref(a), code, vec, ctypes.c_void_p(stream))
        if rc != 0:
            raise RuntimeError(f"generated forward kernel failed to launch (cuda error {rc})")
        counters.bump("flexsn_forward")
        return outs, seqs, last

    def backward(self, inputs, states, seqs, g_outs, g_seqs, g_last, needs: Sequence[bool]):
        """Gradients w.r.t. ``(inputs..., initial states...)``; entries not in ``needs`` are ``None``."""
        from .. import counters
        T, n, code = self._check(inputs, states)
        x0 = inputs[0]
        cont = lambda ts: [None if t is None else t.contiguous() for t in ts]
        g_outs, g_seqs, g_last = cont(g_outs), cont(g_seqs), cont(g_last)
        g_in = [torch.empty_like(x) if needs[i] else None for i, x in enumerate(inputs)]
        g_s0 = [torch.empty_like(s) if needs[self.NI + j] else None for j, s in enumerate(states)]
        if T == 0 or n == 0:
            for j, g in enumerate(g_s0):
                if g is not None:
                    g.zero_() if g_last[j] is None else g.copy_(g_last[j])
            return g_in + g_s0
        a = self._Bwd()
        self._fill(a.inp, inputs)
        self._fill(a.s0, states)
        self._fill(a.s_seq, seqs)
        self._fill(a.g_out, g_outs)
        self._fill(a.g_seq, g_seqs)
        self._fill(a.g_last, g_last)
        self._fill(a.g_in, g_in)
        self._fill(a.g_s0, g_s0)
        a.n, a.T = n, T
        vec = self._vec([*inputs, *states, *seqs, *g_outs, *g_seqs, *g_last, *g_in, *g_s0], n, x0.element_size())
        with _on_device(x0.device):
            stream = torch.cuda.current_stream(x0.device).cuda_stream
            rc = self.lib.flexsn_backward(ctypes.byref(a), code, vec, ctypes.c_void_p(stream))
        if rc != 0:
            raise RuntimeError(f"generated backward kernel failed to launch (cuda error {rc})")
        counters.bump("flexsn_backward")
        return g_in + g_s0


def build_kernel(core: Callable, num_inputs: int, num_states: int, num_outputs: int,
                 example_inputs=None, requires_grad=None, training: bool = True) -> FlexSNKernel:
    graphs = codegen.trace_step(core, num_inputs, num_states, num_outputs, example_inputs, requires_grad, training)
    lib = compiler.compile_module(codegen.emit_module(graphs), name=getattr(core, "__name__", "core"))
    return FlexSNKernel(graphs, lib)


# ----------------------------------------------------------------------- handle registry
_registry_lock = threading.Lock()
_registry: Dict[int, List] = {}          # handle -> [kernel, refcount]
_next_handle = 1


def register_kernel_handle(kernel: FlexSNKernel) -> int:
    global _next_handle
    with _registry_lock:
        h = _next_handle
        _next_handle += 1
        _registry[h] = [kernel, 1]
        return h


def retain_kernel_handle(handle: int) -> None:
    with _registry_lock:
        _registry[handle][1] += 1


def release_kernel_handle(handle: int) -> None:
    with _registry_lock:
        entry = _registry.get(handle)
        if entry is None:
            return
        entry[1] -= 1
        if entry[1] <= 0:
            del _registry[handle]


def lookup_kernel_handle(handle: int) -> FlexSNKernel:
    with _registry_lock:
        entry = _registry.get(int(handle))
    if entry is None:
        raise KeyError(f"neuron kernel handle {handle} is not registered (released, or created in another process)")
    return entry[0]


def attach_handle_finalizer(owner, handle: int):
    """Releases ``handle`` when ``owner`` is collected."""
    return weakref.finalize(owner, release_kernel_handle, handle)


# ----------------------------------------------------------------------- operators
@torch.library.custom_op("sjb200_flexsn::forward", mutates_args=())
def _op_forward(handle: int, args: List[torch.Tensor], store_state_seqs: bool) -> List[torch.Tensor]:
    k = lookup_kernel_handle(handle)
    outs, seqs, last = k.forward(args[:k.NI], args[k.NI:], store_state_seqs)
    return [*outs, *(seqs or []), *last]


@_op_forward.register_fake
def _(handle, args, store_state_seqs):
    k = lookup_kernel_handle(handle)
    x0 = args[0]
    res = [torch.empty_like(x0) for _ in range(k.NO + (k.NS if store_state_seqs else 0))]
    return res + [x0.new_empty(x0.shape[1:]) for _ in range(k.NS)]


@torch.library.custom_op("sjb200_flexsn::backward", mutates_args=())
def _op_backward(handle: int, args: List[torch.Tensor], seqs: List[torch.Tensor], grads: List[Optional[torch.Tensor]],
                 needs: List[bool]) -> List[torch.Tensor]:
    k = lookup_kernel_handle(handle)
    g_outs, g_seqs, g_last = grads[:k.NO], grads[k.NO:k.NO + k.NS], grads[k.NO + k.NS:]
    res = k.backward(args[:k.NI], args[k.NI:], seqs, g_outs, g_seqs, g_last, needs)
    return [r if r is not None else args[0].new_empty(0) for r in res]


@_op_backward.register_fake
def _(handle, args, seqs, grads, needs):
    return [torch.empty_like(a) if n else a.new_empty(0) for a, n in zip(args, needs)]


def flexsn_forward(handle: int, flat_args: Sequence[torch.Tensor], store_state_seqs: bool):
    """No-grad path: ``(outputs, state sequences | None, final states)``."""
    k = lookup_kernel_handle(handle)
    res = _forward_flat(handle, list(flat_args), store_state_seqs)
    outs = res[:k.NO]
    seqs = res[k.NO:k.NO + k.NS] if store_state_seqs else None
    return outs, seqs, res[len(res) - k.NS:]


class _Training(torch.autograd.Function):
    @staticmethod
    def forward(ctx, handle, *flat_args):
        k = lookup_kernel_handle(handle)
        res = _forward_flat(handle, list(flat_args), True)
        seqs = res[k.NO:k.NO + k.NS]
        ctx.kernel = k          # a strong reference: backward works after the module released its handle
        ctx.needs = [bool(n and ctx.needs_input_grad[i + 1]) for i, n in enumerate(k.graphs.needs_grad)]
        ctx.save_for_backward(*flat_args, *seqs)
        ctx.n_args = len(flat_args)
        return tuple(res)

    @staticmethod
    def backward(ctx, *grads):
        saved = ctx.saved_tensors
        args, seqs = list(saved[:ctx.n_args]), list(saved[ctx.n_args:])
        k = ctx.kernel
        res = k.backward(args[:k.NI], args[k.NI:], seqs, grads[:k.NO], grads[k.NO:k.NO + k.NS], grads[k.NO + k.NS:], ctx.needs)
        return (None, *res)


def flexsn_training(handle: int, flat_args: Sequence[torch.Tensor]):
    """Differentiable path: ``(outputs, state sequences, final states)``; the state sequences double as the
    tensors saved for backward."""
    k = lookup_kernel_handle(handle)
    res = _Training.apply(handle, *flat_args)
    return list(res[:k.NO]), list(res[k.NO:k.NO + k.NS]), list(res[k.NO + k.NS:])
