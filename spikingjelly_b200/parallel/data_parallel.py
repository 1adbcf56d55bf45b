"""Data parallelism with gradient all-reduce fused into one kernel per bucket and overlapped
with backward.

:class:`SNNDataParallel` keeps DistributedDataParallel's contract (parameters broadcast from
rank 0 at construction, gradients averaged across ranks by the time ``backward`` returns, module
reachable as ``.module``) but owns the communication:

* gradients live in flat fp32 **symmetric-memory buckets** (parameters are assigned to buckets in
  reverse registration order, like DDP, so that buckets fill in the order backward produces
  them; the bucket that fills LAST — the first layers' parameters — is kept small because its
  exchange cannot hide behind any remaining backward work);
* when the last gradient of a bucket exists, the gradients are gathered into the bucket with one
  multi-tensor copy and a high-priority side stream launches the fused
  ``reduce + scale(1/world) + broadcast`` kernel for that bucket (peer loads/stores over NVLink,
  or in-switch multimem) while the compute stream continues with backward; ``param.grad`` then
  becomes a view of the bucket;
* the end of backward makes the compute stream wait for the side stream and queues a copy of the
  communication status word into pinned host memory.

Failure handling: a peer wait that runs out (``timeout_s``) does not hang the GPU; the kernel skips
the exchange and leaves a status record.  The record is looked at without synchronising at the start
of every ``forward``, by the optimizer hook installed with :meth:`SNNDataParallel.guard_optimizer`
and in :meth:`SNNDataParallel.check_communication` (synchronising); each raises
:class:`~spikingjelly_b200.parallel.comm.CommError`.

``prepare_snn_data_parallel`` has the reference's signature
(``spikingjelly/activation_based/distributed/data_parallel.py:14-35``).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.nn.parallel import DistributedDataParallel

from .comm import CommStatusWord, SymmetricBucket

__all__ = ["SNNDataParallel", "prepare_snn_data_parallel", "unwrap_parallel_module", "materialize_dtensor_output",
           "plan_buckets"]


def plan_buckets(sizes: Sequence[int], cap: int, tail_cap: int) -> List[List[int]]:
    """Group parameter indices (given in registration order with their element counts) into buckets.

    Buckets are filled in reverse registration order up to ``cap`` elements.  The parameters registered
    first (whose gradients arrive last) are split off into a final bucket of at most ``tail_cap``
    elements, so that the exchange which nothing can overlap is short.  Returns lists of indices into
    ``sizes``, in launch order."""
    order = list(range(len(sizes)))[::-1]
    tail: List[int] = []
    n = 0
    while order and n + sizes[order[-1]] <= tail_cap and len(order) > 1:
        n += sizes[order[-1]]
        tail.append(order.pop())
    groups: List[List[int]] = []
    cur: List[int] = []
    cur_n = 0
    for i in order:
        if cur and cur_n + sizes[i] > cap:
            groups.append(cur)
            cur, cur_n = [], 0
        cur.append(i)
        cur_n += sizes[i]
    if cur:
        groups.append(cur)
    if tail:
        groups.append(tail[::-1])
    return groups


class _Bucket:
    def __init__(self, params: List[nn.Parameter], device, group, use_multimem, timeout_s, wire, blocks, status):
        self.params = params
        self.offsets, off = [], 0
        for p in params:
            self.offsets.append(off)
            off += (p.numel() + 3) // 4 * 4        # keep every view 16-byte aligned
        self.sym = SymmetricBucket(off, device, group, use_multimem, timeout_s, wire=wire, blocks=blocks, status=status)
        self.views = [self.sym.buffer[o:o + p.numel()].view_as(p) for o, p in zip(self.offsets, params)]
        self.pending = len(params)
        self.event = torch.cuda.Event() if torch.device(device).type == "cuda" else None


class SNNDataParallel(nn.Module):
    def __init__(self, module: nn.Module, process_group: Optional[dist.ProcessGroup] = None,
                 bucket_cap_mb: float = 25.0, broadcast_buffers: bool = False, use_multimem: Optional[bool] = None,
                 timeout_s: float = 300.0, wire: str = "fp32", blocks: Optional[int] = None,
                 tail_bucket_mb: float = 1.0, reduce: str = "mean"):
        super().__init__()
        if reduce not in ("mean", "sum"):
            raise ValueError(f"reduce must be 'mean' (data parallel) or 'sum' (replicated parameters of a token-sharded model), got {reduce!r}")
        self.reduce = reduce
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
        src = dist.get_global_rank(self.group, 0) if hasattr(dist, "get_global_rank") else 0
        with torch.no_grad():
            for t in list(module.parameters()) + list(module.buffers()):
                dist.broadcast(t, src=src, group=self.group)
        self.status = CommStatusWord(self.device, timeout_s)
        plan = plan_buckets([p.numel() for p in params], int(bucket_cap_mb * (1 << 20) / 4),
                            int(tail_bucket_mb * (1 << 20) / 4))
        self.buckets = [_Bucket([params[i] for i in g], self.device, self.group, use_multimem, timeout_s, wire, blocks,
                                self.status) for g in plan]
        self._where = {}
        self._hooks = []
        for b in self.buckets:
            for i, p in enumerate(b.params):
                self._where[p] = (b, i)
                p.grad = b.views[i]           # gradients accumulate straight into the bucket
                self._hooks.append(p.register_post_accumulate_grad_hook(self._on_grad))
        if self._cuda:
            low, high = torch.cuda.Stream.priority_range()
            self._comm_stream = torch.cuda.Stream(self.device, priority=high)
        else:
            self._comm_stream = None
        self._callback_queued = False
        self._enabled = True

    # ------------------------------------------------------------------ hooks
    def _on_grad(self, p: nn.Parameter) -> None:
        if not self._enabled:
            return
        if not self._callback_queued:
            self._callback_queued = True
            torch.autograd.Variable._execution_engine.queue_callback(self._finish_backward)
        b, _ = self._where[p]
        b.pending -= 1
        if b.pending == 0:
            self._launch(b)

    @staticmethod
    def _gather(b: _Bucket) -> None:
        """Move gradients that autograd left outside the bucket (``zero_grad(set_to_none=True)`` drops the
        views, so the next backward allocates fresh tensors) into it with ONE multi-tensor copy, and
        point ``.grad`` at the views again.  Parameters without a gradient contribute zeros."""
        dst, src = [], []
        for v, p in zip(b.views, b.params):
            g = p.grad
            if g is None:
                v.zero_()
            elif g.data_ptr() != v.data_ptr():
                dst.append(v)
                src.append(g)
        if dst:
            torch._foreach_copy_(dst, src)
        for v, p in zip(b.views, b.params):
            if p.grad is not v and p.grad is not None:
                p.grad = v

    def _launch(self, b: _Bucket) -> None:
        scale = 1.0 / self.world if self.reduce == "mean" else 1.0
        self._gather(b)
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
        launched = False
        for b in self.buckets:
            if b.pending != 0 and b.pending != len(b.params):
                # some parameters of the bucket received no gradient this step: reduce what is there
                self._launch(b)
            if b.pending != len(b.params):
                launched = True
                if self._cuda:
                    torch.cuda.current_stream().wait_event(b.event)
            b.pending = len(b.params)
        if launched and self.world > 1:
            self.status.mirror(self._comm_stream)

    # ------------------------------------------------------------------- API
    def forward(self, *args, **kwargs):
        self.status.poll()
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

    def guard_optimizer(self, optimizer: torch.optim.Optimizer, strict: bool = False):
        """Make ``optimizer.step()`` refuse to run on gradients of a failed exchange.

        ``strict=False`` looks at the pinned status mirror (no synchronisation; sees a failure as soon as
        the host has observed the end of that backward, e.g. after reading the loss).  ``strict=True``
        waits for the exchange of this step to finish first, which serialises host and device once per
        step but guarantees that no update is applied after a failed exchange.  Returns the hook handle."""
        def _pre_step(opt, args, kwargs):
            self.status.poll(wait=strict)
        return optimizer.register_step_pre_hook(_pre_step)

    def release(self) -> None:
        """Remove the gradient hooks and detach ``.grad`` from the buckets (the wrapped module can then be
        wrapped again, e.g. with other exchange settings)."""
        for h in self._hooks:
            h.remove()
        self._hooks = []
        for b in self.buckets:
            for p in b.params:
                p.grad = None

    def check_communication(self) -> None:
        """Synchronise and raise :class:`~spikingjelly_b200.parallel.comm.CommError` if a peer wait expired."""
        if self.world > 1:
            self.status.check()

    @property
    def uses_multimem(self) -> bool:
        return any(b.sym.uses_multimem for b in self.buckets)

    def describe(self) -> dict:
        """Bucket layout and exchange settings (for logs and benchmarks)."""
        return {"world": self.world, "wire": self.buckets[0].sym.wire, "multimem": self.uses_multimem,
                "buckets": [{"params": len(b.params), "numel": b.sym.numel, "blocks": b.sym.blocks,
                             "wire_bytes": b.sym.wire_bytes()} for b in self.buckets]}


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
