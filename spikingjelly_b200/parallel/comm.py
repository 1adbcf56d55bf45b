"""Symmetric-memory gradient buckets and the fused (reduce + scale + broadcast) all-reduce.

A :class:`SymmetricBucket` is a flat fp32 buffer that exists at the same size on every rank and
that every rank can address directly over NVLink (``torch.distributed._symmetric_memory`` supplies
the peer mapping and, where NVSwitch multicast is available, the multimem mapping).
``all_reduce_`` launches ONE kernel (``csrc/comm_allreduce.cu``) on the current stream.

Wire formats: ``"fp32"`` exchanges the bucket itself; ``"bf16"`` keeps the fp32 bucket local and
exchanges a bf16 staging copy (cast, fp32-accumulating reduction, broadcast and widening all inside
the same kernel), which halves the NVLink bytes at the price of bf16 rounding of the summands and
of the mean.

Failure reporting: every device-side wait on a peer is bounded by ``timeout_s``.  A wait that runs
out leaves a record in a :class:`CommStatusWord`; the word is mirrored into pinned host memory
without blocking (:meth:`CommStatusWord.mirror`) so the training loop can look at it before every
step at the cost of one host-memory read (:meth:`CommStatusWord.poll`).

Without CUDA (unit tests on ``gloo``) the same interface falls back to ``dist.all_reduce``.
"""
from __future__ import annotations

import os
from typing import List, Optional

import torch
import torch.distributed as dist

__all__ = ["SymmetricBucket", "CommStatusWord", "CommError", "next_epoch", "EPOCH_MASK"]

#: the device compares flags and epochs as wrapping 32-bit counters (``(int32)(flag - epoch) >= 0``),
#: so the host counter wraps modulo 2^32 as well
EPOCH_MASK = 0xFFFFFFFF


def next_epoch(epoch: int, step: int) -> int:
    """The epoch counter after one collective that consumes ``step`` epochs (wraps modulo 2^32)."""
    return (epoch + step) & EPOCH_MASK


def epoch_reached(flag: int, epoch: int) -> bool:
    """Host restatement of the device predicate ``(int32_t)(flag - epoch) >= 0`` on uint32 counters."""
    d = (flag - epoch) & EPOCH_MASK
    return d < 0x80000000


class CommError(RuntimeError):
    """A bounded device-side wait on a peer expired (the peer never reached the collective)."""


class CommStatusWord:
    """``{code, rank, peer, block}`` written by a collective kernel whose wait ran out, plus a pinned
    host mirror that can be read without synchronising."""

    def __init__(self, device: torch.device, timeout_s: float):
        self.device = torch.device(device)
        self.timeout_s = float(timeout_s)
        self.dev = torch.zeros(4, dtype=torch.int32, device=self.device)
        pinned = self.device.type == "cuda"
        self.host = torch.zeros(4, dtype=torch.int32, pin_memory=pinned)
        self._event = torch.cuda.Event() if pinned else None

    def mirror(self, stream: Optional["torch.cuda.Stream"] = None) -> None:
        """Queue a non-blocking copy of the device word into the host mirror (after everything already
        queued on ``stream``)."""
        if self.device.type != "cuda":
            self.host.copy_(self.dev)
            return
        stream = stream or torch.cuda.current_stream(self.device)
        with torch.cuda.stream(stream):
            self.host.copy_(self.dev, non_blocking=True)
            self._event.record(stream)

    def poll(self, wait: bool = False) -> None:
        """Raise :class:`CommError` if the host mirror shows a failed wait.  ``wait=True`` first blocks
        until the last queued mirror copy has landed (a device synchronisation point); ``wait=False``
        is a plain host-memory read and may lag behind the device by the work still in flight."""
        if wait and self._event is not None:
            self._event.synchronize()
        code = int(self.host[0])
        if code == 0:
            return
        _, rank, peer, block = (int(v) for v in self.host)
        self.host.zero_()
        self.dev.zero_()
        phase = "waiting for the peer's bucket" if code == 1 else "waiting for the peer's results"
        raise CommError(f"rank {rank}: a fused collective gave up {phase} from rank {peer} (block {block}) after "
                        f"{self.timeout_s:.1f} s; gradients of that step were not reduced")

    def check(self) -> None:
        """Synchronising check of the device word itself."""
        self.mirror()
        self.poll(wait=True)


def _auto_blocks(numel: int, world: int, multimem: bool) -> int:
    """Blocks per kernel.  Every thread keeps about eight 16-byte accesses in flight, so a block of 512 threads
    covers 64 KB per round trip; 16 blocks (1 MB in flight) are enough to fill the link, and small buckets need
    fewer.  Few blocks leave the SMs to the backward kernels that run concurrently.  With ``multimem`` the switch
    reduces and one request returns the sum of all ranks: 4 to 8 blocks already give the best time measured at eight
    GPUs (95 us for a 25 MB bucket), more only take SMs."""
    slice_bytes = 4 * numel / max(world, 1)
    want = int(slice_bytes // (128 << 10)) + 1
    return max(2, min(8 if multimem else 16, want))


class SymmetricBucket:
    #: upper bound of the per-kernel block count (sizes the signal pad)
    MAX_BLOCKS = 64

    def __init__(self, numel: int, device: torch.device, group: Optional[dist.ProcessGroup] = None,
                 use_multimem: Optional[bool] = None, timeout_s: float = 300.0, wire: str = "fp32",
                 blocks: Optional[int] = None, status: Optional[CommStatusWord] = None):
        if wire not in ("fp32", "bf16"):
            raise ValueError(f"wire must be 'fp32' or 'bf16', got {wire!r}")
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.numel = (numel + 7) // 8 * 8
        self.timeout_s = float(timeout_s)
        self.device = torch.device(device)
        self.wire = wire
        self._epoch = 1
        self._native = self.device.type == "cuda" and self.world > 1
        self.status = status if status is not None else CommStatusWord(self.device, timeout_s)
        if use_multimem is None:
            env = os.environ.get("SJB200_DP_MULTIMEM")
            use_multimem = None if env is None else env not in ("0", "false", "no")
        if self._native:
            from .. import ops
            import torch.distributed._symmetric_memory as symm
            ops.require()
            self.buffer = symm.empty(self.numel, dtype=torch.float32, device=self.device)
            self._signal = symm.empty(self.MAX_BLOCKS * self.world, dtype=torch.int32, device=self.device)
            self.buffer.zero_()
            self._signal.zero_()
            h_sig = symm.rendezvous(self._signal, self.group)
            self._sig_ptrs: List[int] = [int(p) for p in h_sig.buffer_ptrs]
            if wire == "bf16":
                self._stage = symm.empty(self.numel, dtype=torch.bfloat16, device=self.device)
                self._stage.zero_()
                h_buf = symm.rendezvous(self._stage, self.group)
            else:
                self._stage = None
                h_buf = symm.rendezvous(self.buffer, self.group)
            self._buf_ptrs: List[int] = [int(p) for p in h_buf.buffer_ptrs]
            # multicast_ptr is 0 where the fabric offers no NVSwitch multicast mapping
            mc = int(getattr(h_buf, "multicast_ptr", 0) or 0)
            self._mc_ptr = mc if (use_multimem is None or use_multimem) else 0
            self._handles = (h_buf, h_sig)
            self.blocks = int(blocks) if blocks else _auto_blocks(self.numel, self.world, self._mc_ptr != 0)
            if not 1 <= self.blocks <= self.MAX_BLOCKS:
                raise ValueError(f"blocks must be in [1, {self.MAX_BLOCKS}]")
            torch.cuda.synchronize(self.device)
            dist.barrier(self.group)          # every peer has zeroed its flags before anyone signals
        else:
            self.buffer = torch.zeros(self.numel, dtype=torch.float32, device=self.device)
            self._mc_ptr = 0
            self.blocks = 0

    @property
    def uses_multimem(self) -> bool:
        return self._mc_ptr != 0

    def wire_bytes(self) -> int:
        """Bytes one rank sends (and receives) over NVLink per all-reduce: (world-1)/world of the bucket in
        the reduce phase plus the same in the broadcast phase."""
        elt = 2 if self.wire == "bf16" else 4
        return int(2 * self.numel * elt * (self.world - 1) / self.world)

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
                                              self._epoch, float(scale), self.blocks, self.status.dev, self.timeout_s,
                                              1 if self.wire == "bf16" else 0)
            self._epoch = next_epoch(self._epoch, 2)
            return
        dist.all_reduce(self.buffer, group=self.group)
        if scale != 1.0:
            self.buffer.mul_(scale)

    def check(self) -> None:
        """Synchronises and raises :class:`CommError` if a peer wait expired since the last check."""
        if self._native:
            self.status.check()
