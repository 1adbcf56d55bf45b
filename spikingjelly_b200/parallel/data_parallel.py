"""Data parallelism with gradient all-reduce fused into one kernel per bucket and overlapped
with backward.

:class:`SNNDataParallel` keeps DistributedDataParallel's contract (parameters broadcast from
rank 0 at construction, gradients averaged across ranks by the time ``backward`` returns, module
reachable as ``.module``) but owns the communication:

* gradients live in flat fp32 **symmetric-memory buckets** (parameters are assigned to buckets in
  reverse registration order, like DDP, so that buckets fill in the order backward produces
  them); ``param.grad`` is a view of its bucket;
* when the last gradient of a bucket has been accumulated, a side stream launches the fused
  ``reduce + scale(1/world) + broadcast`` kernel for that bucket (peer loads/stores over NVLink,
  or in-switch multimem) while the compute stream continues with backward;
* the end of backward makes the compute stream wait for the side stream.

``prepare_snn_data_parallel`` has the reference's signature
(``spikingjelly/activation_based/distributed/data_parallel.py:14-35``).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.nn.parallel import DistributedDataParallel

from .comm import SymmetricBucket

__all__ = ["SNNDataParallel", "prepare_snn_data_parallel", "unwrap_parallel_module", "materialize_dtensor_output"]


class _Bucket:
    def __init__(self, params: List[nn.Parameter], device, group, use_multimem, timeout_s):
        self.params = params
        self.offsets, off = [], 0
        for p in params:
            self.offsets.append(off)
            off += (p.numel() + 3) // 4 * 4        # keep every view 16-byte aligned
        self.sym = SymmetricBucket(off, device, group, use_multimem, timeout_s)
        self.views = [self.sym.buffer[o:o + p.numel()].view_as(p) for o, p in zip(self.offsets, params)]
        self.pending = len(params)
        self.event = torch.cuda.Event() if torch.device(device).type == "cuda" else None


class SNNDataParallel(nn.Module):
    def __init__(self, module: nn.Module, process_group: Optional[dist.ProcessGroup] = None,
                 bucket_cap_mb: float = 25.0, broadcast_buffers: bool = False, use_multimem: bool = False,
                 timeout_s: float = 2.0):
        super().__init__()
        self.module = module
        self.group = process_group if process_group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.broadcast_buffers = broadcast_buffers
        params = [p for p in module.parameters() if p.requires_grad]
        if not params:
            raise ValueError("SNNDataParallel needs at least one parameter that requires grad")
        self.device = params[0].device
        self._cuda = self.device.type == "cuda"
        # same initial weights everywhere
        with torch.no_grad():
            for t in list(module.parameters()) + list(module.buffers()):
                dist.broadcast(t, src=dist.get_global_rank(self.group, 0) if hasattr(dist, "get_global_rank") else 0,
                               group=self.group)
        # reverse registration order, capped buckets
        cap = int(bucket_cap_mb * (1 << 20) / 4)
        groups, cur, cur_n = [], [], 0
        for p in reversed(params):
            if cur and cur_n + p.numel() > cap:
                groups.append(cur)
                cur, cur_n = [], 0
            cur.append(p)
            cur_n += p.numel()
        if cur:
            groups.append(cur)
        self.buckets = [_Bucket(g, self.device, self.group, use_multimem, timeout_s) for g in groups]
        self._where = {}
        for b in self.buckets:
            for i, p in enumerate(b.params):
                self._where[p] = (b, i)
                p.grad = b.views[i]           # gradients accumulate straight into the bucket
                p.register_post_accumulate_grad_hook(self._on_grad)
        self._comm_stream = torch.cuda.Stream(self.device) if self._cuda else None
        self._callback_queued = False
        self._enabled = True

    # ------------------------------------------------------------------ hooks
    def _on_grad(self, p: nn.Parameter) -> None:
        if not self._enabled:
            return
        if not self._callback_queued:
            self._callback_queued = True
            torch.autograd.Variable._execution_engine.queue_callback(self._finish_backward)
        b, i = self._where[p]
        if p.grad is not b.views[i]:
            # the optimizer dropped the view (zero_grad(set_to_none=True)): move the fresh gradient
            # into the bucket and point .grad at the view again
            b.views[i].copy_(p.grad)
            p.grad = b.views[i]
        b.pending -= 1
        if b.pending == 0:
            self._launch(b)

    def _launch(self, b: _Bucket) -> None:
        scale = 1.0 / self.world
        if self._cuda:
            ready = torch.cuda.Event()
            ready.record()                                   # gradients of this bucket are final here
            with torch.cuda.stream(self._comm_stream):
                self._comm_stream.wait_event(ready)
                b.sym.all_reduce_(scale)
                b.event.record()
        else:
            b.sym.all_reduce_(scale)

    def _finish_backward(self) -> None:
        self._callback_queued = False
        for b in self.buckets:
            if b.pending != 0 and b.pending != len(b.params):
                # some parameters of the bucket received no gradient this step: reduce what is there
                self._launch(b)
            if self._cuda and b.pending != len(b.params):
                torch.cuda.current_stream().wait_event(b.event)
            b.pending = len(b.params)

    # ------------------------------------------------------------------- API
    def forward(self, *args, **kwargs):
        if self.broadcast_buffers and self.world > 1:
            with torch.no_grad():
                for t in self.module.buffers():
                    dist.broadcast(t, src=0, group=self.group)
        return self.module(*args, **kwargs)

    def no_sync(self):
        """Context manager: accumulate gradients locally (no all-reduce) inside the block."""
        outer = self

        class _Ctx:
            def __enter__(self_inner):
                outer._enabled = False

            def __exit__(self_inner, *exc):
                outer._enabled = True
        return _Ctx()

    def check_communication(self) -> None:
        """Raise :class:`~spikingjelly_b200.parallel.comm.CommError` if a peer wait expired."""
        for b in self.buckets:
            b.sym.check()

    @property
    def uses_multimem(self) -> bool:
        return any(b.sym.uses_multimem for b in self.buckets)


def prepare_snn_data_parallel(module: nn.Module, process_group=None, device_ids: Optional[Sequence[int]] = None,
                              broadcast_buffers: bool = False, find_unused_parameters: bool = False,
                              static_graph: bool = False, fused: bool = True, **kwargs):
    """Wrap ``module`` for data-parallel training.  ``fused=True`` (default) returns
    :class:`SNNDataParallel`; ``fused=False`` returns ``torch``'s DistributedDataParallel (NCCL
    all-reduce), which is also what is used when some parameters may receive no gradient
    (``find_unused_parameters``)."""
    if fused and not find_unused_parameters:
        return SNNDataParallel(module, process_group, broadcast_buffers=broadcast_buffers, **kwargs)
    return DistributedDataParallel(module, device_ids=list(device_ids) if device_ids is not None else None,
                                   process_group=process_group, broadcast_buffers=broadcast_buffers,
                                   find_unused_parameters=find_unused_parameters, static_graph=static_graph)


def unwrap_parallel_module(module: nn.Module) -> nn.Module:
    return module.module if isinstance(module, (DistributedDataParallel, SNNDataParallel)) else module


def materialize_dtensor_output(output):
    """Gather sharded (DTensor-like: anything with ``full_tensor()``) outputs, recursively through
    tuples, named tuples, lists and dicts; other values pass through."""
    full = getattr(output, "full_tensor", None)
    if callable(full):
        return full()
    if isinstance(output, tuple):
        items = [materialize_dtensor_output(o) for o in output]
        return output.__class__(*items) if hasattr(output, "_fields") else tuple(items)
    if isinstance(output, list):
        return [materialize_dtensor_output(o) for o in output]
    if isinstance(output, dict):
        return {k: materialize_dtensor_output(v) for k, v in output.items()}
    return output
