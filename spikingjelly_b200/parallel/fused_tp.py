"""Sequence-sharded tensor parallelism for spike-driven transformer blocks with the collectives inside the GEMMs.

The residual stream ``h`` is split by tokens over the group (rank ``r`` holds ``h[:, r * n : (r + 1) * n]``).
One fused sub-layer ``h += W2 . LIF(W1 . LIF(RMSNorm(h)))`` with ``W1`` split by rows and ``W2`` by columns runs as

1. ``rmsnorm_lif_pack``: norm + LIF over T on the local tokens; the spikes leave the kernel as bits, stored into
   the gather buffer of EVERY rank (16-byte peer stores: the all-gather is the producer's epilogue and moves 1/16
   of the bf16 payload, once per peer);
2. barrier; ``spike_gemm`` (gather): every rank multiplies ALL tokens by its rows of ``W1`` — the A-operand producer
   of the GEMM expands the 1-bit rows of all source ranks from its local gather buffer (the kernel takes one
   pointer per source rank, so it can also read the peers' buffers in place; measured on two GPUs that costs
   the NVLink latency once per n-tile and is slower than the push);
3. ``lif_pack``: LIF over T on the local columns, bits stay local;
4. ``spike_gemm`` (push): partial products of ``W2`` leave the epilogue as peer stores into the owner's staging slot
   (reduce-scatter inside the epilogue);
5. barrier; ``tp_reduce_residual``: the owner adds the slots in rank order onto its shard of ``h``.

All kernels are in ``ops/csrc/tp_fused.cu``; waits on peers are bounded and surface as :class:`CommError`.  The path
is forward-only (serving, evaluation, activation statistics): training uses ``parallel.tensor_parallel``.
With one rank the same kernels run on local buffers, which is how the single-GPU tests exercise them.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .comm import CommError, next_epoch

__all__ = ["FusedTPWorkspace", "FusedSpikingSubLayer", "pack_pitch", "fused_ffn_from_block"]


def pack_pitch(columns: int) -> int:
    """Bytes per packed row: 1 bit per column, padded to a multiple of 32 bytes."""
    return (columns + 255) // 256 * 32


def _pad_to(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class FusedTPWorkspace:
    """Symmetric buffers shared by every fused sub-layer of a model (they run one after another)."""

    def __init__(self, T: int, tokens_per_rank: int, d_model: int, device, group: Optional[dist.ProcessGroup] = None,
                 timeout_s: float = 120.0):
        if tokens_per_rank % 128 or d_model % 256:
            raise ValueError("tokens_per_rank must be a multiple of 128 and d_model a multiple of 256")
        self.T, self.tokens_per_rank, self.d_model = T, tokens_per_rank, d_model
        self.device = torch.device(device)
        self.timeout_s = float(timeout_s)
        distributed = dist.is_available() and dist.is_initialized()
        self.group = group if group is not None else (dist.group.WORLD if distributed else None)
        self.world = dist.get_world_size(self.group) if distributed else 1
        self.rank = dist.get_rank(self.group) if distributed else 0
        self.rows = T * tokens_per_rank
        self.x_pitch = pack_pitch(d_model)
        self.slot_elems = self.rows * d_model
        self._epoch = 1
        from .. import ops
        ops.require()
        if self.world > 1:
            import torch.distributed._symmetric_memory as symm
            self.bits_x = symm.empty(self.world * self.rows * self.x_pitch, dtype=torch.uint8, device=self.device)
            self.stage = symm.empty(self.world * self.slot_elems, dtype=torch.bfloat16, device=self.device)
            self._signal = symm.empty(self.world, dtype=torch.int32, device=self.device)
            for t in (self.bits_x, self.stage, self._signal):
                t.zero_()
            hb, hs, hg = (symm.rendezvous(t, self.group) for t in (self.bits_x, self.stage, self._signal))
            slot = self.rows * self.x_pitch                      # one source rank's packed rows
            # the GEMM reads source s from the local slot s; this rank's pack kernel writes slot `rank` everywhere
            self.bits_ptrs: List[int] = [self.bits_x.data_ptr() + s * slot for s in range(self.world)]
            self.bits_push_ptrs: List[int] = [int(p) + self.rank * slot for p in hb.buffer_ptrs]
            self.stage_ptrs: List[int] = [int(p) for p in hs.buffer_ptrs]
            self.sig_ptrs: List[int] = [int(p) for p in hg.buffer_ptrs]
            self._handles = (hb, hs, hg)
            torch.cuda.synchronize(self.device)
            dist.barrier(self.group)
        else:
            self.bits_x = torch.zeros(self.rows * self.x_pitch, dtype=torch.uint8, device=self.device)
            self.stage = torch.zeros(self.slot_elems, dtype=torch.bfloat16, device=self.device)
            self._signal = torch.zeros(1, dtype=torch.int32, device=self.device)
            self.bits_ptrs, self.stage_ptrs, self.sig_ptrs = [self.bits_x.data_ptr()], [self.stage.data_ptr()], [self._signal.data_ptr()]
            self.bits_push_ptrs = [self.bits_x.data_ptr()]
        self._status = torch.zeros(4, dtype=torch.int32, device=self.device)
        self._local_bits: dict = {}

    def local_bits(self, columns: int) -> torch.Tensor:
        """Scratch for the packed spikes of a column-parallel output: all tokens x ``columns`` bits."""
        buf = self._local_bits.get(columns)
        if buf is None:
            buf = torch.zeros(self.T * self.tokens_per_rank * self.world * pack_pitch(columns), dtype=torch.uint8, device=self.device)
            self._local_bits[columns] = buf
        return buf

    def barrier(self) -> None:
        """Every rank's earlier kernels are complete and their peer stores visible.  One tiny kernel."""
        if self.world == 1:
            return
        torch.ops.sjb200.tp_barrier(self.sig_ptrs, self.rank, self._epoch, self._status, self.timeout_s)
        self._epoch = next_epoch(self._epoch, 1)

    def check(self) -> None:
        """Synchronises; raises if a peer wait or a pipeline wait inside a GEMM expired since the last check."""
        code, rank, peer, _ = self._status.tolist()
        if code != 0:
            self._status.zero_()
            raise CommError(f"rank {rank}: fused tensor-parallel barrier gave up waiting for rank {peer} after {self.timeout_s:.1f} s")
        st = torch.ops.sjb200.gemm_status(self._status)
        if st[0] != 0:
            raise RuntimeError(f"spike_gemm pipeline wait expired (code {st[0]}, block {st[1]}, detail {st[2]})")


class FusedSpikingSubLayer(nn.Module):
    """``h += W2 . LIF(W1 . LIF(RMSNorm(h)))`` on a token-sharded residual stream (bias-free linears).

    ``w1``: full ``[F, d]`` weight, split by rows; ``w2``: full ``[d, F]``, split by columns.  The local ``F / world``
    slice is zero-padded to a multiple of 256 so that packed rows keep their 32-byte pitch (the padded neurons
    never fire)."""

    def __init__(self, ws: FusedTPWorkspace, norm_weight: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, eps: float = 1e-6,
                 tau: float = 2.0, v_threshold: float = 1.0):
        super().__init__()
        self.ws, self.eps, self.tau, self.v_threshold = ws, float(eps), float(tau), float(v_threshold)
        F, d = w1.shape
        if d != ws.d_model or tuple(w2.shape) != (d, F) or F % ws.world:
            raise ValueError("weights must be [F, d] and [d, F] with F divisible by the group size")
        fl = F // ws.world
        self.f_local, self.f_pad = fl, _pad_to(fl, 256)
        lo = ws.rank * fl
        dev = ws.device
        w1p = torch.zeros(self.f_pad, d, dtype=torch.bfloat16, device=dev)
        w1p[:fl] = w1[lo:lo + fl].to(dev, torch.bfloat16)
        w2p = torch.zeros(d, self.f_pad, dtype=torch.bfloat16, device=dev)
        w2p[:, :fl] = w2[:, lo:lo + fl].to(dev, torch.bfloat16)
        self.register_buffer("w1", w1p)
        self.register_buffer("w2", w2p)
        self.register_buffer("norm_weight", norm_weight.detach().to(dev, torch.float32).contiguous())

    @torch.no_grad()
    def forward(self, h: torch.Tensor) -> torch.Tensor:
        """``h``: ``[T, tokens_per_rank, d]`` fp32 or bf16, contiguous; updated in place and returned."""
        ws = self.ws
        if tuple(h.shape) != (ws.T, ws.tokens_per_rank, ws.d_model) or not h.is_contiguous():
            raise ValueError(f"expected a contiguous [{ws.T}, {ws.tokens_per_rank}, {ws.d_model}] tensor")
        ops = torch.ops.sjb200
        tokens = ws.tokens_per_rank * ws.world
        M = ws.T * tokens
        ops.rmsnorm_lif_pack(h, self.norm_weight, ws.bits_push_ptrs, ws.x_pitch, self.eps, self.tau, self.v_threshold)
        ws.barrier()                                             # everybody's spikes are in place
        u = ops.spike_gemm(ws.bits_ptrs, ws.x_pitch, M, ws.d_model, self.w1, tokens, ws.tokens_per_rank, ws.rank, [], 0)
        bits_u = ws.local_bits(self.f_pad)
        pitch_u = pack_pitch(self.f_pad)
        ops.lif_pack(u.view(ws.T, tokens, self.f_pad), bits_u.data_ptr(), pitch_u, self.tau, self.v_threshold)
        ops.spike_gemm([bits_u.data_ptr()], pitch_u, M, self.f_pad, self.w2, tokens, ws.tokens_per_rank, ws.rank,
                       ws.stage_ptrs, ws.slot_elems)
        ws.barrier()                                             # every partial product has landed
        ops.tp_reduce_residual(h, ws.stage.data_ptr(), ws.slot_elems, ws.world)
        return h

    @torch.no_grad()
    def reference(self, h_full: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor) -> torch.Tensor:
        """The same arithmetic with plain PyTorch on the unsharded problem (fp32 LIF, bf16 matmul operands)."""
        return _reference_sublayer(h_full, self.norm_weight, w1, w2, self.eps, self.tau, self.v_threshold)


def _lif_seq(x: torch.Tensor, tau: float, v_th: float) -> torch.Tensor:
    v = torch.zeros_like(x[0])
    out = []
    inv = torch.tensor(1.0 / tau, dtype=torch.float32).item()
    for t in range(x.shape[0]):
        hh = v + (x[t] - v) * inv
        s = (hh >= v_th).to(x.dtype)
        v = hh * (1 - s)
        out.append(s)
    return torch.stack(out)


def _reference_sublayer(h, norm_w, w1, w2, eps, tau, v_th):
    hf = h.float()
    x = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps) * norm_w.float()
    s = _lif_seq(x, tau, v_th)
    u = (s.to(torch.bfloat16) @ w1.to(h.device, torch.bfloat16).t()).float()      # the GEMM rounds its result to bf16
    su = _lif_seq(u, tau, v_th)
    y = su.to(torch.bfloat16).float() @ w2.to(h.device, torch.bfloat16).float().t()
    return hf + y


def fused_ffn_from_block(block, ws: FusedTPWorkspace) -> FusedSpikingSubLayer:
    """The FFN half of an :class:`~spikingjelly_b200.models.snn_llm.SNNLLMBlock` as a fused sub-layer."""
    cfg = block.attn.cfg
    return FusedSpikingSubLayer(ws, block.norm2.weight, block.ffn.up.weight, block.ffn.down.weight, cfg.rms_eps, cfg.tau, 1.0)
