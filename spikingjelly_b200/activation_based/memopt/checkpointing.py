"""Gradient checkpointing that stores a *compressed* copy of the segment input.

``input_compressed_gc(f, compressor, x, *args)`` runs ``f`` without building a graph, keeps only
``compressor.compress(x)`` (plus the other tensor arguments, RNG and autocast state), and in
backward decompresses, re-runs ``f`` with the saved RNG/autocast state and back-propagates.
``GCContainer`` / ``TCGCContainer`` are ``nn.Sequential`` wrappers around it; the latter also
splits the time axis into chunks.  Stateful modules are supported by threading their memories
through the checkpointed function explicitly (``base.to_functional_forward``).

Parity: ``spikingjelly/activation_based/memopt/checkpointing.py:25-602``.
"""
from __future__ import annotations

import contextlib
import functools
import threading
from typing import Any, Callable, Optional, Tuple

import torch
import torch.nn as nn

from ...logger import logger
from .. import base
from .compress import BaseSpikeCompressor, NullSpikeCompressor

__all__ = ["in_gc_1st_forward", "query_autocast", "input_compressed_gc", "to_gc_function", "GCContainer",
           "TCGCContainer", "InputCompressedGC"]

_tls = threading.local()


@contextlib.contextmanager
def _discarded_forward():
    depth = getattr(_tls, "depth", 0)
    _tls.depth = depth + 1
    try:
        yield
    finally:
        _tls.depth = depth


def in_gc_1st_forward() -> bool:
    """True while a checkpointed segment runs its first (graph-free) forward; BatchNorm layers
    use it to skip the running-statistics update that the recomputation will perform."""
    return getattr(_tls, "depth", 0) > 0


def query_autocast() -> Tuple[str, torch.dtype, bool]:
    for dev in ("cuda", "cpu"):
        if torch.is_autocast_enabled(dev):
            return dev, torch.get_autocast_dtype(dev), True
    return "cpu", torch.get_autocast_dtype("cpu"), False


class InputCompressedGC(torch.autograd.Function):
    @staticmethod
    def forward(ctx, f_forward: Callable, x_compressor: BaseSpikeCompressor, x_seq, *args):
        ctx.f_forward, ctx.x_compressor, ctx.x_shape = f_forward, x_compressor, x_seq.shape
        ctx.autocast = query_autocast()
        stored = (x_compressor.compress(x_seq), *args)
        ctx.is_tensor = [torch.is_tensor(a) for a in stored]
        ctx.others = [None if t else a for a, t in zip(stored, ctx.is_tensor)]
        ctx.save_for_backward(*[a for a, t in zip(stored, ctx.is_tensor) if t])
        ctx.rng_cpu = torch.get_rng_state()
        ctx.rng_cuda = torch.cuda.get_rng_state_all() if torch.cuda.is_initialized() else []
        with _discarded_forward(), torch.no_grad():
            return f_forward(x_seq, *args)

    @staticmethod
    def backward(ctx, *grad_outputs):
        grads = [None] * (len(ctx.is_tensor) + 2)
        if not any(ctx.needs_input_grad):
            return tuple(grads)
        saved = iter(ctx.saved_tensors)
        stored = [next(saved) if t else o for t, o in zip(ctx.is_tensor, ctx.others)]
        packed, args = stored[0], stored[1:]
        dev, dt, on = ctx.autocast
        with torch.enable_grad(), torch.autocast(dev, dt, on):
            x = ctx.x_compressor.decompress(packed, ctx.x_shape).detach().requires_grad_(True)
            for i, a in enumerate(args):
                if torch.is_tensor(a):
                    args[i] = a.detach().requires_grad_(bool(ctx.needs_input_grad[3 + i] and a.requires_grad))
            with torch.random.fork_rng(range(torch.cuda.device_count()) if ctx.rng_cuda else []):
                torch.set_rng_state(ctx.rng_cpu)
                if ctx.rng_cuda:
                    torch.cuda.set_rng_state_all(ctx.rng_cuda)
                outputs = ctx.f_forward(x, *args)
        if isinstance(outputs, torch.Tensor):
            outputs = (outputs,)
        pairs = [(o, g) for o, g in zip(outputs, grad_outputs) if torch.is_tensor(o) and o.requires_grad]
        torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        if ctx.needs_input_grad[2]:
            grads[2] = x.grad
        for i, a in enumerate(args):
            if ctx.needs_input_grad[3 + i] and torch.is_tensor(a):
                grads[3 + i] = a.grad
        return tuple(grads)


def input_compressed_gc(f_forward, x_compressor: BaseSpikeCompressor, x_seq, *args):
    """Checkpoint ``f_forward(x_seq, *args)``, storing ``x_seq`` compressed.  Plain call without grad."""
    if not torch.is_grad_enabled():
        return f_forward(x_seq, *args)
    if not x_seq.requires_grad:
        x_seq = x_seq.detach().requires_grad_(True)     # the output must be attached to the graph
    return InputCompressedGC.apply(f_forward, x_compressor, x_seq, *args)


def to_gc_function(x_compressor: BaseSpikeCompressor, f_forward: Optional[Callable] = None):
    """Decorator (or converter) turning ``f(x_seq, *args)`` into its checkpointed version."""
    def decorate(fn):
        @functools.wraps(fn)
        def wrapped(x_seq, *args):
            return input_compressed_gc(fn, x_compressor, x_seq, *args)
        return wrapped
    return decorate if f_forward is None else decorate(f_forward)


class GCContainer(nn.Sequential):
    """``nn.Sequential`` whose forward is checkpointed with a compressed input."""

    def __init__(self, x_compressor: Optional[BaseSpikeCompressor], *args):
        super().__init__(*args)
        self.x_compressor = NullSpikeCompressor() if x_compressor is None else x_compressor
        self._bind()

    def _bind(self):
        self.f_forward = base.to_functional_forward(self, fn=self.super_forward)
        self.num_states = len(list(base.memories(self)))

    def __getstate__(self):
        state = self.__dict__.copy()
        state.pop("f_forward", None)
        return state

    def __setstate__(self, state):
        self.__dict__.update(state)
        self._bind()

    def super_forward(self, *inputs: Any) -> Any:
        out = inputs
        for m in self:
            r = m(*out)
            out = tuple(r) if isinstance(r, (tuple, list)) else (r,)
        return out[0] if len(out) == 1 else out

    def stateless_forward(self, x, *args):
        return input_compressed_gc(self.super_forward, self.x_compressor, x, *args)

    def stateful_forward(self, x, *args):
        states = tuple(base.extract_memories(self))
        n_in = 1 + len(args)

        def flat(*flat_args):
            outs, new_states = self.f_forward(tuple(flat_args[:n_in]), tuple(flat_args[n_in:]))
            return (*outs, *new_states)

        ret = input_compressed_gc(flat, self.x_compressor, x, *args, *states)
        outs, new_states = ret[:-self.num_states], ret[-self.num_states:]
        base.load_memories(self, list(new_states))
        return outs[0] if len(outs) == 1 else outs

    def forward(self, x, *args):
        if len(list(base.memories(self))) != self.num_states:
            self._bind()
        return self.stateful_forward(x, *args) if self.num_states else self.stateless_forward(x, *args)

    def extra_repr(self) -> str:
        return f"x_compressor={self.x_compressor.__class__.__name__},"


class TCGCContainer(GCContainer):
    """Temporal chunking + checkpointing: the first ``n_seq_inputs`` inputs are split into
    ``n_chunk`` pieces along time, each piece is checkpointed on its own, outputs are concatenated."""

    def __init__(self, x_compressor: Optional[BaseSpikeCompressor], *args, n_chunk: int = 1, n_seq_inputs: int = 1,
                 n_outputs: int = 1):
        super().__init__(x_compressor, *args)
        self.n_chunk, self.n_seq_inputs, self.n_outputs = n_chunk, n_seq_inputs, n_outputs

    def forward(self, x_seq, *args):
        n_chunk = min(self.n_chunk, x_seq.shape[0])
        if n_chunk != self.n_chunk:
            logger.warning("TCGCContainer received n_chunk=%d for sequence length T=%d; using n_chunk=%d.",
                           self.n_chunk, x_seq.shape[0], n_chunk)
        seqs = (x_seq, *args[: self.n_seq_inputs - 1])
        rest = args[self.n_seq_inputs - 1:]
        pieces = [torch.tensor_split(s, n_chunk, dim=0) for s in seqs]
        collected = [[] for _ in range(self.n_outputs)]
        for i in range(n_chunk):
            outs = super().forward(*[p[i] for p in pieces], *rest)
            outs = outs if isinstance(outs, tuple) else (outs,)
            for bucket, o in zip(collected, outs):
                bucket.append(o)
        final = [torch.cat(c, dim=0) for c in collected]
        return final[0] if len(final) == 1 else tuple(final)

    def extra_repr(self):
        return (f"x_compressor={self.x_compressor.__class__.__name__}, n_chunk={self.n_chunk}, "
                f"n_seq_inputs={self.n_seq_inputs}, n_seq_outputs={self.n_outputs}")
