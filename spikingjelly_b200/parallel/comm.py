"""Symmetric-memory gradient buckets and the fused (reduce + scale + broadcast) all-reduce.

A :class:`SymmetricBucket` is a flat fp32 buffer that exists at the same size on every rank and
that every rank can address directly over NVLink (``torch.distributed._symmetric_memory`` supplies
the peer mapping and, where NVSwitch multicast is available, the multimem mapping).
``all_reduce_`` launches ONE kernel (``csrc/comm_allreduce.cu``) on the current stream.

Without CUDA (unit tests on ``gloo``) the same interface falls back to ``dist.all_reduce``.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

__all__ = ["SymmetricBucket", "CommError"]


class CommError(RuntimeError):
    """A bounded device-side wait on a peer expired (the peer never reached the collective)."""


class SymmetricBucket:
    #: blocks per all-reduce kernel: enough to saturate NVLink, few enough to leave SMs to the
    #: backward kernels that run concurrently on the compute stream
    BLOCKS = 32

    def __init__(self, numel: int, device: torch.device, group: Optional[dist.ProcessGroup] = None,
                 use_multimem: bool = False, timeout_s: float = 2.0):
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.numel = (numel + 3) // 4 * 4
        self.timeout_s = float(timeout_s)
        self.device = torch.device(device)
        self._epoch = 1
        self._native = self.device.type == "cuda" and self.world > 1
        if self._native:
            from .. import ops
            import torch.distributed._symmetric_memory as symm
            ops.require()
            self.buffer = symm.empty(self.numel, dtype=torch.float32, device=self.device)
            self._signal = symm.empty(self.BLOCKS * self.world, dtype=torch.int32, device=self.device)
            self.buffer.zero_()
            self._signal.zero_()
            h_buf = symm.rendezvous(self.buffer, self.group)
            h_sig = symm.rendezvous(self._signal, self.group)
            self._buf_ptrs: List[int] = [int(p) for p in h_buf.buffer_ptrs]
            self._sig_ptrs: List[int] = [int(p) for p in h_sig.buffer_ptrs]
            # multicast_ptr is 0 where the fabric offers no NVSwitch multicast mapping
            self._mc_ptr = int(h_buf.multicast_ptr or 0) if use_multimem else 0
            self._handles = (h_buf, h_sig)
            self._status = torch.zeros(4, dtype=torch.int32, device=self.device)
            torch.cuda.synchronize(self.device)
            dist.barrier(self.group)          # every peer has zeroed its flags before anyone signals
        else:
            self.buffer = torch.zeros(self.numel, dtype=torch.float32, device=self.device)
            self._mc_ptr = 0

    @property
    def uses_multimem(self) -> bool:
        return self._mc_ptr != 0

    def all_reduce_(self, scale: float) -> None:
        """In place: ``buffer <- scale * sum over ranks(buffer)`` on the current stream."""
        if self.world == 1:
            if scale != 1.0:
                self.buffer.mul_(scale)
            return
        if self._native:
            from ..ops import counters
            counters.bump("allreduce_bucket")
            torch.ops.sjb200.allreduce_bucket(self.buffer, self._buf_ptrs, self._sig_ptrs, self._mc_ptr, self.rank,
                                              self._epoch, float(scale), self.BLOCKS, self._status, self.timeout_s)
            self._epoch = (self._epoch + 2) & 0x7FFFFFFF
            return
        dist.all_reduce(self.buffer, group=self.group)
        if scale != 1.0:
            self.buffer.mul_(scale)

    def check(self) -> None:
        """Synchronises and raises :class:`CommError` if a peer wait expired since the last check."""
        if not self._native:
            return
        code, rank, peer, block = self._status.tolist()
        if code != 0:
            self._status.zero_()
            phase = "waiting for the peer's bucket" if code == 1 else "waiting for the peer's results"
            raise CommError(f"rank {rank}: all-reduce gave up {phase} from rank {peer} (block {block}) "
                            f"after {self.timeout_s:.1f} s")
