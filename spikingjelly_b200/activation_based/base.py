"""Core runtime: step modes, stateful modules and the functional-state protocol.

Behavioural parity with ``spikingjelly/activation_based/base.py``:
``StepModule`` (:99-210), ``SingleStepModule``/``MultiStepModule`` (:213-310),
``MemoryModule`` (:313-1125), the free helpers ``named_memories`` / ``memories`` /
``extract_memories`` / ``load_memories`` (:1128-1312) and
``to_functional_forward`` (:1315-1551).

Backends.  There are two execution paths: ``"torch"`` (eager PyTorch ops, works on
any device and is the numerical oracle) and ``"cuda"`` (hand-written sm_100a
kernels from :mod:`spikingjelly_b200.ops`).  The reference's backend names
``"cupy"``, ``"triton"`` and ``"inductor"`` are accepted everywhere and resolve to
``"cuda"`` so that existing scripts keep working.
"""
from __future__ import annotations

import copy
from typing import Any, Callable, Generator, Optional, Tuple

import torch
import torch.nn as nn

from ..logger import logger

__all__ = [
    "check_backend_library", "canonical_backend", "StepModule", "SingleStepModule",
    "MultiStepModule", "MemoryModule", "ElidedState", "elide_states", "named_memories", "memories",
    "extract_memories", "load_memories", "to_functional_forward",
]

_NATIVE_ALIASES = ("cuda", "cupy", "triton", "inductor")


def canonical_backend(name: str) -> str:
    """Map a user-facing backend string to the path that will run it."""
    return "cuda" if name in _NATIVE_ALIASES else name


def check_backend_library(backend: str) -> None:
    """Raise ``ImportError`` if ``backend`` cannot run in this process.

    ``"torch"`` always can.  The native path needs the compiled extension; it is
    only *loaded* lazily on first use on a CUDA tensor, so this check succeeds on
    CPU-only hosts as long as the extension source tree is present.
    ``"lava"`` needs Lava-DL.  Parity: ``base.py:35-96``.
    """
    backend = canonical_backend(backend)
    if backend in ("torch", "cuda"):
        return
    if backend == "lava":
        try:
            import lava.lib.dl.slayer  # noqa: F401
        except (ImportError, OSError) as exc:
            raise ImportError("Lava-DL is not installed (https://github.com/lava-nc/lava-dl).") from exc


class StepModule:
    """Mixin that gives a module a ``step_mode``: ``"s"`` consumes one time step
    ``[N, *]``, ``"m"`` consumes a whole sequence ``[T, N, *]``."""

    def supported_step_mode(self) -> Tuple[str, ...]:
        return ("s", "m")

    @property
    def step_mode(self) -> str:
        return self._step_mode

    @step_mode.setter
    def step_mode(self, value: str) -> None:
        if value not in self.supported_step_mode():
            raise ValueError(f'step_mode can only be {self.supported_step_mode()}, but got "{value}"!')
        self._step_mode = value


class SingleStepModule(StepModule):
    def supported_step_mode(self):
        return ("s",)


class MultiStepModule(StepModule):
    def supported_step_mode(self):
        return ("m",)


def _same_layout(a: Any, b: Any) -> bool:
    return (isinstance(a, torch.Tensor) and isinstance(b, torch.Tensor) and a.shape == b.shape
            and a.dtype == b.dtype and a.device == b.device)


class ElidedState:
    """Placeholder memory value: "this state was advanced by a fused schedule that does not keep it".

    The fused model schedules start every sequence from the reset state and never write the membrane potentials
    back.  They leave this marker in the neurons' memories so that a second forward without ``reset()`` fails loudly
    (the module path would carry the state over; silently restarting from the reset value would not).  ``reset()``
    and ``load_memories`` replace it like any other value."""

    def __repr__(self):
        return "ElidedState()"


def elide_states(modules) -> None:
    """Mark every memory of the given :class:`MemoryModule` instances as not kept (see :class:`ElidedState`)."""
    for m in modules:
        for key in m._memories:
            m._memories[key] = ElidedState()


class MemoryModule(nn.Module, StepModule):
    """A module with resettable state ("memories", e.g. membrane potential ``v``).

    Memories live in ``self._memories`` (never in ``state_dict``); each has a reset
    value in ``self._memories_rv``.  ``self.<name>`` reads/writes the dict.  A Python
    scalar as memory is a *sentinel*: the first forward materialises it to a tensor
    shaped like the input, and ``reset()`` puts the scalar back so that the next
    input may have another shape.

    Subclasses implement the pure ``single_step_functional_forward(inputs, states)
    -> (outputs, states)``; the stateful ``forward`` is derived from it.
    """

    def __init__(self):
        super().__init__()
        self._memories: dict = {}
        self._memories_rv: dict = {}
        self._backend = "torch"
        self._step_mode = "s"

    # ------------------------------------------------------------------ backend
    @property
    def supported_backends(self) -> Tuple[str, ...]:
        return ("torch",)

    @property
    def backend(self) -> str:
        return self._backend

    @backend.setter
    def backend(self, value: str) -> None:
        supported = self.supported_backends
        if value not in supported and canonical_backend(value) not in supported:
            raise NotImplementedError(f"{value} is not a supported backend of {self._get_name()}!")
        check_backend_library(value)
        self._backend = value

    @property
    def native(self) -> bool:
        """True when the configured backend resolves to the sm_100a kernels."""
        return canonical_backend(self._backend) == "cuda"

    # ------------------------------------------------- functional-state protocol
    def materialize_states(self, inputs: tuple, states: tuple, step_mode: str) -> tuple:
        """Turn sentinel states into tensors that match ``inputs``.  Identity here."""
        return states

    def single_step_functional_forward(self, inputs: tuple, states: tuple, **kwargs):
        raise NotImplementedError(f"{self._get_name()} does not implement single_step_functional_forward.")

    def multi_step_functional_forward(self, inputs: tuple, states: tuple, **kwargs):
        """Default: walk the leading time axis with the single-step rule."""
        collected = None
        for t in range(inputs[0].shape[0]):
            outs, states = self.single_step_functional_forward(tuple(x[t] for x in inputs), states, **kwargs)
            if collected is None:
                collected = [[] for _ in outs]
            if len(outs) != len(collected):
                raise ValueError("single_step_functional_forward changed its number of outputs")
            for bucket, o in zip(collected, outs):
                bucket.append(o)
        return tuple(torch.stack(b) for b in (collected or [])), states

    def functional_forward(self, inputs: tuple, states: tuple, **kwargs):
        mode = self.step_mode
        if mode not in ("s", "m"):
            raise ValueError(mode)
        states = self.materialize_states(inputs, states, mode)
        if mode == "s":
            return self.single_step_functional_forward(inputs, states, **kwargs)
        return self.multi_step_functional_forward(inputs, states, **kwargs)

    # ------------------------------------------------------------ stateful calls
    def _commit(self, new_states: tuple) -> None:
        names = list(self._memories.keys())
        if len(names) != len(new_states):
            raise ValueError(f"{self._get_name()} has {len(names)} memories but got {len(new_states)} states")
        for n, s in zip(names, new_states):
            self._memories[n] = s

    def single_step_forward(self, x: torch.Tensor, *args, **kwargs):
        inputs = (x, *args)
        states = self.materialize_states(inputs, tuple(self._memories.values()), "s")
        outs, new_states = self.single_step_functional_forward(inputs, states, **kwargs)
        self._commit(new_states)
        return outs[0] if len(outs) == 1 else outs

    def multi_step_forward(self, x_seq: torch.Tensor, *args, **kwargs):
        inputs = (x_seq, *args)
        states = self.materialize_states(inputs, tuple(self._memories.values()), "m")
        outs, new_states = self.multi_step_functional_forward(inputs, states, **kwargs)
        self._commit(new_states)
        return outs[0] if len(outs) == 1 else outs

    def forward(self, *args, **kwargs):
        for value in self._memories.values():
            if isinstance(value, ElidedState):
                raise RuntimeError(
                    f"{type(self).__name__}: a fused model schedule advanced this module without storing its state; "
                    "call functional.reset_net() before the next forward, or set `model.fused = False` for stateful use")
        if self.step_mode == "s":
            return self.single_step_forward(*args, **kwargs)
        if self.step_mode == "m":
            return self.multi_step_forward(*args, **kwargs)
        raise ValueError(self.step_mode)

    def extra_repr(self):
        return f"step_mode={self.step_mode}, backend={self.backend}"

    # ----------------------------------------------------------------- memories
    def register_memory(self, name: str, value) -> None:
        assert not hasattr(self, name), f"{name} has been set as a member variable!"
        self._memories[name] = value
        self.set_reset_value(name, value)

    def set_reset_value(self, name: str, value) -> None:
        self._memories_rv[name] = copy.deepcopy(value)

    def get_reset_value(self, name: str) -> Any:
        if name not in self._memories:
            raise KeyError(f"{name} is not a registered memory.")
        if name not in self._memories_rv:
            raise KeyError(f"{name} has no reset value. Call set_reset_value first.")
        return self._memories_rv[name]

    def reset(self) -> None:
        """Restore every memory to its reset value (in place when the layout matches,
        so that CUDA-graph captured buffers stay valid)."""
        for key, cur in self._memories.items():
            rv = self._memories_rv[key]
            if _same_layout(cur, rv):
                try:
                    cur.detach_()
                except RuntimeError:  # views cannot be detached in place
                    self._memories[key] = rv.detach().clone()
                else:
                    cur.copy_(rv)
            elif isinstance(cur, torch.Tensor) and isinstance(rv, (int, float)):
                self._memories[key] = rv
            else:
                self._memories[key] = copy.deepcopy(rv)

    def detach(self) -> None:
        """Cut the autograd history of all tensor memories (truncated BPTT)."""
        for value in self._memories.values():
            if isinstance(value, torch.Tensor):
                value.detach_()

    def memories(self) -> Generator:
        yield from self._memories.values()

    def named_memories(self) -> Generator:
        yield from self._memories.items()

    def __getattr__(self, name: str):
        mem = self.__dict__.get("_memories")
        if mem is not None and name in mem:
            return mem[name]
        return super().__getattr__(name)

    def __setattr__(self, name: str, value) -> None:
        mem = self.__dict__.get("_memories")
        if mem is not None and name in mem:
            mem[name] = value
        else:
            super().__setattr__(name, value)

    def __delattr__(self, name):
        if name in self._memories:
            del self._memories[name]
            del self._memories_rv[name]
        else:
            super().__delattr__(name)

    def __dir__(self):
        keys = (dir(self.__class__) + list(self.__dict__) + list(self._parameters) + list(self._modules)
                + list(self._buffers) + list(self._memories))
        return sorted(k for k in set(keys) if not k[0].isdigit())

    def _apply(self, fn, *args, **kwargs):
        for key, value in self._memories.items():
            if isinstance(value, torch.Tensor):
                self._memories[key] = fn(value)
        return super()._apply(fn, *args, **kwargs)

    def _replicate_for_data_parallel(self):
        replica = super()._replicate_for_data_parallel()
        replica._memories = self._memories.copy()
        return replica


# ----------------------------------------------------------------- tree helpers
def named_memories(module: nn.Module, prefix: str = "") -> Generator:
    """Yield ``(dotted_name, value)`` for every memory below ``module`` (pre-order)."""
    if isinstance(module, MemoryModule):
        for name, value in module.named_memories():
            yield (f"{prefix}.{name}" if prefix else name), value
    for child_name, child in module.named_children():
        yield from named_memories(child, f"{prefix}.{child_name}" if prefix else child_name)


def memories(module: nn.Module) -> Generator:
    for _, value in named_memories(module):
        yield value


def extract_memories(module: nn.Module) -> list:
    return list(memories(module))


def load_memories(module: nn.Module, memory_list: list) -> None:
    """Inverse of :func:`extract_memories` (same traversal order)."""
    names = [n for n, _ in named_memories(module)]
    if len(names) != len(memory_list):
        raise ValueError(f"Memory length mismatch: model has {len(names)} memories but list contains {len(memory_list)}")
    for name, value in zip(names, memory_list):
        *path, leaf = name.split(".")
        owner = module
        for p in path:
            owner = getattr(owner, p)
        setattr(owner, leaf, value)


def _overrides_functional(m: "MemoryModule") -> bool:
    cls = type(m)
    if cls.functional_forward is not MemoryModule.functional_forward:
        return True
    if cls.single_step_functional_forward is not MemoryModule.single_step_functional_forward:
        return True
    return m.step_mode == "m" and cls.multi_step_functional_forward is not MemoryModule.multi_step_functional_forward


def _as_tuple(x) -> tuple:
    return tuple(x) if isinstance(x, (tuple, list)) else (x,)


def to_functional_forward(module: nn.Module, fn: Optional[Callable] = None) -> Callable:
    """Build ``f(inputs, states, **kw) -> (outputs, new_states)`` from ``module``.

    ``states`` is the flat tuple in :func:`extract_memories` order.  Three
    strategies, fastest first: (1) a single MemoryModule that implements the
    functional protocol is called directly; (2) a flat ``nn.Sequential`` is
    composed child by child, threading states without touching module memory;
    (3) anything else: load ``states`` into the modules, run ``fn`` (default: the
    module's own forward), read the new states back, and restore the previous
    memories so that the call is pure from the outside.
    """
    mem_modules = [m for m in module.modules() if isinstance(m, MemoryModule)]
    n_states = sum(len(m._memories) for m in mem_modules)

    def _check(states):
        if len(states) != n_states:
            raise ValueError(f"{module.__class__.__name__} expected {n_states} states, but got {len(states)}.")

    if fn is None and isinstance(module, MemoryModule) and len(mem_modules) == 1 and _overrides_functional(module):
        def direct(inputs, states, **kwargs):
            _check(states)
            return module.functional_forward(inputs, states, **kwargs)
        return direct

    if fn is None and isinstance(module, nn.Sequential):
        children = list(module._modules.values())
        counts = [len(c._memories) if isinstance(c, MemoryModule) and _overrides_functional(c) else 0 for c in children]
        if sum(counts) == n_states:
            def chained(inputs, states, **kwargs):
                _check(states)
                cur, new_states, ofs = inputs, [], 0
                for i, (child, cnt) in enumerate(zip(children, counts)):
                    kw = kwargs if i == 0 else {}
                    if cnt:
                        cur, upd = child.functional_forward(cur, states[ofs:ofs + cnt], **kw)
                        new_states.extend(upd)
                        ofs += cnt
                    else:
                        cur = _as_tuple(child(*cur, **kw))
                return cur, tuple(new_states)
            return chained

    call = fn if fn is not None else module

    def swapped(inputs, states, **kwargs):
        _check(states)
        saved = extract_memories(module)
        try:
            load_memories(module, list(states))
            outputs = _as_tuple(call(*inputs, **kwargs))
            new_states = tuple(extract_memories(module))
        finally:
            load_memories(module, saved)
        return outputs, new_states

    return swapped
