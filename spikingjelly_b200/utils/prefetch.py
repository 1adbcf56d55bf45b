"""Input pipeline helpers that keep the GPU busy between training steps.

``DevicePrefetcher`` copies the NEXT batch from pinned host memory on a side stream while the current step computes;
``DeferredScalar`` reads a device scalar (the loss) back without stalling the launch of the following step: the copy is
queued behind the step, and the value is picked up one step later.  Both degrade to plain synchronous behaviour on CPU.

    pf = DevicePrefetcher(device)
    staged = pf.stage(x_host, y_host)
    for i in range(steps):
        x, y = pf.take(staged)
        if i + 1 < steps:
            staged = pf.stage(next_x_host, next_y_host)
        loss = train_step(x, y)
        reader = DeferredScalar(loss)            # D2H copy queued
        if previous is not None:
            log(previous.get())                  # value of the step before: ready by now
        previous = reader
"""
from __future__ import annotations

from typing import Tuple

import torch

__all__ = ["DevicePrefetcher", "DeferredScalar"]


class DevicePrefetcher:
    def __init__(self, device):
        self.device = torch.device(device)
        self.stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None

    def stage(self, *host_tensors: torch.Tensor):
        """Start the copies; returns a token for :meth:`take`."""
        if self.stream is None:
            return tuple(t.to(self.device) for t in host_tensors), None
        with torch.cuda.stream(self.stream):
            out = tuple(t.to(self.device, non_blocking=True) for t in host_tensors)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        return out, ev

    def take(self, staged) -> Tuple[torch.Tensor, ...]:
        """Make the current stream wait for the staged copies and hand the tensors over to it."""
        out, ev = staged
        if ev is not None:
            cur = torch.cuda.current_stream(self.device)
            cur.wait_event(ev)
            for t in out:
                t.record_stream(cur)
        return out


class DeferredScalar:
    """``DeferredScalar(t)`` queues a device-to-host copy of the one-element tensor ``t``; ``get()`` waits for it."""

    # Pinned landing buffers are reused in turn (a first pinned allocation costs milliseconds and may synchronise the
    # device); eight cover every loop that reads a value at most seven steps late.
    _ring: dict = {}
    _cursor = 0
    _RING = 8

    def __init__(self, value: torch.Tensor):
        v = value.detach().reshape(1)
        if v.is_cuda:
            cls = DeferredScalar
            ring = cls._ring.setdefault(v.dtype, [])
            if len(ring) < cls._RING:
                ring.append(torch.empty(1, dtype=v.dtype, pin_memory=True))
            self._host = ring[cls._cursor % len(ring)]
            cls._cursor += 1
            self._host.copy_(v, non_blocking=True)
            self._event = torch.cuda.Event()
            self._event.record(torch.cuda.current_stream(v.device))
        else:
            self._host, self._event = v.clone(), None

    def get(self) -> float:
        if self._event is not None:
            self._event.synchronize()
        return float(self._host.item())
