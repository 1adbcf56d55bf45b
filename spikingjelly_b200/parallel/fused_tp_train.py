"""Training through the fused tensor-parallel path: forward AND backward of a spike-driven transformer block with the
collectives inside (or directly around) this package's own kernels, no NCCL on the activation path.

The residual stream is sharded by tokens (rank ``r`` owns tokens ``[r n, (r + 1) n)`` of the flattened batch).  A sub-layer is

    h  +=  Row( mid( Col( LIF(RMSNorm(h)) ) ) )

with ``Col`` a column-parallel linear (rows of the weight split over the ranks: FFN up projection, QKV by whole heads),
``Row`` a row-parallel linear (FFN down, attention output) and ``mid`` a local function (LIF for the FFN; rotary embedding,
causal attention and LIF for the attention sub-layer).  The four communication patterns are

======================  ===========================================  ==========================================
pass                    what crosses NVLink                          how
======================  ===========================================  ==========================================
``Col`` forward         the input spikes, 1 bit each (all-gather)    ``bit_pack`` -> ``tp_push_chunks`` (peer stores into every
                                                                     rank's ``[T][tokens][d / 8]`` buffer) -> ``spike_gemm``,
                                                                     whose A-operand producer expands the bits
``Row`` forward         partial products (reduce-scatter)            epilogue of ``spike_gemm`` stores each tile into its owner's
                                                                     staging slot; the owner adds the slots in rank order
``Row`` backward        output gradients, bf16 (all-gather)          ``tp_push_chunks`` -> tcgen05 GEMMs on the gathered rows
``Col`` backward        partial input gradients (reduce-scatter)     tcgen05 GEMM into a symmetric buffer -> ``tp_reduce_chunks``
                                                                     (each owner reads its rows from every peer and adds them)
======================  ===========================================  ==========================================

so one sub-layer moves ``1/16 + 1`` activation-sized messages forward and ``2`` backward, against eight for the all-reduce
formulation (two all-reduces each way, each a reduce-scatter plus an all-gather).  Weight gradients need no communication:
every rank sees the gradients of ALL tokens for its slice of the weights.  Saved for backward: the gathered input spikes and
the local hidden spikes as bits, and the pre-activation of the middle LIF.

Peer memory is touched only by this package's kernels with plain loads / stores; TMA and library kernels see local memory.
Every buffer that a peer writes is guarded by a flag barrier before its next use (bounded waits, :class:`CommError`).

Counterpart in the reference: the DTensor redistributions of ``distributed/tensor_parallel/linear.py:287-392`` and the
hand-written all-reduces of ``distributed/tensor_parallel/channel.py:42-55,153-167``.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..activation_based import neuron, surrogate
from ..ops import bitpack
from ..ops import gemm as G
from .fused_tp import FusedTPWorkspace

__all__ = ["FusedTPTrainWorkspace", "column_parallel_from_spikes", "row_parallel_to_stream", "FusedTPSubLayer",
           "FusedTPSNNLLM"]


def _pad_rows(w: torch.Tensor, rows: int) -> torch.Tensor:
    if w.shape[0] == rows:
        return w.contiguous()
    out = w.new_zeros((rows, w.shape[1]))
    out[:w.shape[0]] = w
    return out


def _pad_cols(w: torch.Tensor, cols: int) -> torch.Tensor:
    if w.shape[1] == cols:
        return w.contiguous()
    out = w.new_zeros((w.shape[0], cols))
    out[:, :w.shape[1]] = w
    return out


class FusedTPTrainWorkspace(FusedTPWorkspace):
    """The forward workspace plus the two symmetric buffers of the backward pass: ``gy`` (gathered output gradients) and
    ``partial`` (this rank's partial input gradients, read by their owners).  One workspace serves every sub-layer of a
    model; they run one after another."""

    def __init__(self, T: int, tokens_per_rank: int, d_model: int, device, group: Optional[dist.ProcessGroup] = None,
                 timeout_s: float = 120.0):
        super().__init__(T, tokens_per_rank, d_model, device, group, timeout_s)
        n_all = self.world * self.slot_elems
        if self.world > 1:
            import torch.distributed._symmetric_memory as symm
            self.gy = symm.empty(n_all, dtype=torch.bfloat16, device=self.device)
            self.partial = symm.empty(n_all, dtype=torch.bfloat16, device=self.device)
            self.gy.zero_()
            self.partial.zero_()
            hy, hp = symm.rendezvous(self.gy, self.group), symm.rendezvous(self.partial, self.group)
            self.gy_ptrs: List[int] = [int(p) for p in hy.buffer_ptrs]
            self.partial_ptrs: List[int] = [int(p) for p in hp.buffer_ptrs]
            self.bits_base_ptrs: List[int] = [int(p) for p in self._handles[0].buffer_ptrs]
            self._train_handles = (hy, hp)
            torch.cuda.synchronize(self.device)
            dist.barrier(self.group)
        else:
            self.gy = torch.zeros(n_all, dtype=torch.bfloat16, device=self.device)
            self.partial = torch.zeros(n_all, dtype=torch.bfloat16, device=self.device)
            self.gy_ptrs, self.partial_ptrs = [self.gy.data_ptr()], [self.partial.data_ptr()]
            self.bits_base_ptrs = [self.bits_x.data_ptr()]

    @property
    def tokens(self) -> int:
        return self.tokens_per_rank * self.world


class _ColumnParallelFromSpikes(torch.autograd.Function):
    @staticmethod
    def forward(ctx, s_local: torch.Tensor, weight: torch.Tensor, ws: FusedTPTrainWorkspace, cols_pad: int):
        T, n, d = s_local.shape
        tokens, M, row = ws.tokens, T * ws.tokens, d // 8
        ops = torch.ops.sjb200
        w = _pad_rows(weight.detach().to(torch.bfloat16), cols_pad)
        bits = bitpack.bit_spike_compress(s_local.detach().contiguous())
        ws.barrier()                                             # everybody is done reading the gather buffer's previous contents
        ops.tp_push_chunks(bits, ws.bits_base_ptrs, T, tokens * row, ws.rank * n * row)
        ws.barrier()                                             # everybody's spikes are in place
        u = ops.spike_gemm([ws.bits_x.data_ptr()], row, M, d, w, tokens, tokens, 0, [], 0)
        ctx.ws, ctx.shape, ctx.rows = ws, (T, n, d), weight.shape[0]
        ctx.in_dtype, ctx.w_dtype = s_local.dtype, weight.dtype
        ctx.save_for_backward(ws.bits_x[:M * row].clone(), w)
        return u.view(T, tokens, cols_pad)

    @staticmethod
    def backward(ctx, g_u: torch.Tensor):
        bits_full, w = ctx.saved_tensors
        ws: FusedTPTrainWorkspace = ctx.ws
        T, n, d = ctx.shape
        tokens, M = ws.tokens, T * ws.tokens
        ops = torch.ops.sjb200
        g2 = g_u.reshape(M, -1).to(torch.bfloat16).contiguous()
        g_s = g_w = None
        if ctx.needs_input_grad[1]:
            s_full = bitpack.bit_spike_decompress(bits_full, (M, d), torch.bfloat16)
            g_w = G.gemm(g2, s_full, True, True, out_f32=True)[:ctx.rows].to(ctx.w_dtype)        # [cols, d]
        if ctx.needs_input_grad[0]:
            ws.barrier()                                         # the owners have read the previous partial sums
            ops.gemm_16bit_into(g2, w, False, True, ws.partial[:M * d].view(M, d))               # all tokens x d, this rank's share
            ws.barrier()
            g_local = torch.empty((T, n, d), dtype=torch.bfloat16, device=g2.device)
            ops.tp_reduce_chunks(ws.partial_ptrs, g_local, T, tokens * d, ws.rank * n * d)
            g_s = g_local.to(ctx.in_dtype)
        return g_s, g_w, None, None


class _RowParallelToStream(torch.autograd.Function):
    @staticmethod
    def forward(ctx, su: torch.Tensor, weight: torch.Tensor, ws: FusedTPTrainWorkspace, cols_pad: int):
        T, tokens, _ = su.shape
        n, d, M = ws.tokens_per_rank, ws.d_model, T * tokens
        ops = torch.ops.sjb200
        w = _pad_cols(weight.detach().to(torch.bfloat16), cols_pad)                              # [d, cols_pad]
        bits = bitpack.bit_spike_compress(su.detach().contiguous())                              # pitch cols_pad / 8
        ws.barrier()                                             # the owners have added up their previous staging slots
        ops.spike_gemm([bits.data_ptr()], cols_pad // 8, M, cols_pad, w, tokens, n, ws.rank, ws.stage_ptrs, ws.slot_elems)
        ws.barrier()                                             # every partial product has landed
        y = torch.zeros((T, n, d), dtype=torch.bfloat16, device=su.device)
        ops.tp_reduce_residual(y, ws.stage.data_ptr(), ws.slot_elems, ws.world)
        ctx.ws, ctx.cols, ctx.cols_pad = ws, weight.shape[1], cols_pad
        ctx.in_dtype, ctx.w_dtype, ctx.T = su.dtype, weight.dtype, T
        ctx.save_for_backward(bits, w)
        return y

    @staticmethod
    def backward(ctx, g_y: torch.Tensor):
        bits, w = ctx.saved_tensors
        ws: FusedTPTrainWorkspace = ctx.ws
        T, tokens, n, d = ctx.T, ws.tokens, ws.tokens_per_rank, ws.d_model
        M = T * tokens
        ops = torch.ops.sjb200
        gy = g_y.to(torch.bfloat16).contiguous()
        ws.barrier()                                             # everybody is done with the previously gathered gradients
        ops.tp_push_chunks(gy, ws.gy_ptrs, T, tokens * d * 2, ws.rank * n * d * 2)
        ws.barrier()
        gy_full = ws.gy[:M * d].view(M, d)
        g_su = g_w = None
        if ctx.needs_input_grad[0]:
            g_su = G.gemm(gy_full, w, False, True).view(T, tokens, ctx.cols_pad).to(ctx.in_dtype)
        if ctx.needs_input_grad[1]:
            su_full = bitpack.bit_spike_decompress(bits, (M, ctx.cols_pad), torch.bfloat16)
            g_w = G.gemm(gy_full, su_full, True, True, out_f32=True)[:, :ctx.cols].to(ctx.w_dtype)   # [d, cols]
        return g_su, g_w, None, None


def column_parallel_from_spikes(s_local: torch.Tensor, weight: torch.Tensor, ws: FusedTPTrainWorkspace, cols_pad: int) -> torch.Tensor:
    """``s_local``: this rank's ``[T, n, d]`` spikes (0 / 1).  ``weight``: this rank's ``[cols, d]`` rows.  Returns the
    pre-activations of ALL tokens for these columns, ``[T, tokens, cols_pad]`` bf16 (columns past ``cols`` are zero)."""
    return _ColumnParallelFromSpikes.apply(s_local, weight, ws, cols_pad)


def row_parallel_to_stream(su: torch.Tensor, weight: torch.Tensor, ws: FusedTPTrainWorkspace, cols_pad: int) -> torch.Tensor:
    """``su``: ``[T, tokens, cols_pad]`` spikes of this rank's columns for all tokens.  ``weight``: this rank's ``[d, cols]``
    columns.  Returns this rank's ``[T, n, d]`` share of the full product (summed over the ranks), bf16."""
    return _RowParallelToStream.apply(su, weight, ws, cols_pad)


def _lif(tau: float) -> neuron.LIFNode:
    return neuron.LIFNode(tau=tau, detach_reset=True, surrogate_function=surrogate.ATan(), step_mode="m", backend="cuda")


class FusedTPSubLayer(nn.Module):
    """``h + Row(mid(Col(LIF(RMSNorm(h)))))`` on a token-sharded stream.  ``w_in``: this rank's rows ``[cols, d]`` of the
    column-parallel weight, ``w_out``: this rank's columns ``[d, cols_out]`` of the row-parallel one.  ``mid`` maps
    ``[T, tokens, cols_pad]`` pre-activations to ``[T, tokens, cols_out_pad]`` spikes (default: a LIF neuron)."""

    def __init__(self, ws: FusedTPTrainWorkspace, norm_weight: torch.Tensor, w_in: torch.Tensor, w_out: torch.Tensor, eps: float,
                 tau: float, mid: Optional[nn.Module] = None):
        super().__init__()
        self.ws, self.eps = ws, float(eps)
        self.norm_weight = nn.Parameter(norm_weight.detach().clone().float())
        self.w_in = nn.Parameter(w_in.detach().clone())
        self.w_out = nn.Parameter(w_out.detach().clone())
        self.cols_pad = (w_in.shape[0] + 255) // 256 * 256
        self.cols_out_pad = (w_out.shape[1] + 255) // 256 * 256
        self.lif_in = _lif(tau)
        self.mid = mid if mid is not None else _lif(tau)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        x = F.rms_norm(h.float(), (h.shape[-1],), self.norm_weight, self.eps).to(torch.bfloat16)
        s = self.lif_in(x)
        u = column_parallel_from_spikes(s, self.w_in, self.ws, self.cols_pad)
        su = self.mid(u)
        y = row_parallel_to_stream(su, self.w_out, self.ws, self.cols_out_pad)
        return h + y.to(h.dtype)


class _AttentionCore(nn.Module):
    """QKV pre-activations of this rank's heads for all tokens -> attention -> LIF spikes (the ``mid`` of the attention
    sub-layer).  Tokens are the flattened ``[batch, sequence]`` order, so a gathered row block is whole sequences."""

    def __init__(self, rope: nn.Module, local_heads: int, head_dim: int, seq_len: int, cols_out_pad: int, tau: float):
        super().__init__()
        self.rope, self.H, self.D, self.S, self.cols_out_pad = rope, local_heads, head_dim, seq_len, cols_out_pad
        self.lif = _lif(tau)

    def forward(self, u: torch.Tensor) -> torch.Tensor:
        from ..ops import rope as rope_ops
        T, tokens, _ = u.shape
        B, H, D, S = tokens // self.S, self.H, self.D, self.S
        qkv = u[..., :3 * H * D].reshape(T * B, S, H, 3, D)
        if rope_ops.supports(qkv, D):
            q, k, v = (t.transpose(1, 2) for t in rope_ops.rope_qkv(qkv, self.rope.cos, self.rope.sin))
            a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        else:
            q, k, v = (qkv[:, :, :, i].transpose(1, 2) for i in range(3))
            a = F.scaled_dot_product_attention(self.rope(q), self.rope(k), v, is_causal=True)
        a = a.transpose(1, 2).reshape(T, tokens, H * D)
        if H * D != self.cols_out_pad:
            a = F.pad(a, (0, self.cols_out_pad - H * D))
        return self.lif(a)


class FusedTPSNNLLM(nn.Module):
    """An :class:`~spikingjelly_b200.models.snn_llm.SNNLLM` re-wired for fused tensor-parallel training.

    Weights of the four linears of every block are sliced for this rank (QKV by whole heads, FFN by columns); embedding,
    norms and LM head stay replicated and see only this rank's tokens, so THEIR gradients must be summed over the group
    after backward (:meth:`replicated_parameters` lists them; wrap them with
    ``SNNDataParallel(..., reduce="sum")`` or all-reduce them).  The loss returned by :meth:`forward` is this rank's share
    ``sum over local tokens / number of predicted tokens in the batch``: the shares add up to the batch loss, and with that
    normalisation the sliced weights receive their exact gradients without further scaling."""

    def __init__(self, model, batch: int, seq_len: int, group: Optional[dist.ProcessGroup] = None, timeout_s: float = 120.0):
        super().__init__()
        cfg = model.cfg
        distributed = dist.is_available() and dist.is_initialized()
        world = dist.get_world_size(group) if distributed else 1
        rank = dist.get_rank(group) if distributed else 0
        tokens = batch * seq_len
        if tokens % world or cfg.n_heads % world or cfg.d_ffn % world:
            raise ValueError(f"batch * seq_len ({tokens}), n_heads ({cfg.n_heads}) and d_ffn ({cfg.d_ffn}) must be divisible by the group size {world}")
        device = model.embed.weight.device
        self.cfg, self.batch, self.seq_len, self.world, self.rank, self.group = cfg, batch, seq_len, world, rank, group
        self.ws = FusedTPTrainWorkspace(cfg.T, tokens // world, cfg.d_model, device, group, timeout_s)
        self.embed, self.norm_f, self.lm_head = model.embed, model.norm_f, model.lm_head
        d, D = cfg.d_model, cfg.head_dim
        hl, fl = cfg.n_heads // world, cfg.d_ffn // world
        layers = []
        for blk in model.blocks:
            wq = blk.attn.qkv.weight.detach()[rank * 3 * hl * D:(rank + 1) * 3 * hl * D]         # rows are head-major: whole heads
            wo = blk.attn.proj.weight.detach()[:, rank * hl * D:(rank + 1) * hl * D]
            core = _AttentionCore(blk.attn.rope, hl, D, seq_len, (hl * D + 255) // 256 * 256, cfg.tau)
            attn = FusedTPSubLayer(self.ws, blk.norm1.weight, wq, wo, cfg.rms_eps, cfg.tau, mid=core)
            ffn = FusedTPSubLayer(self.ws, blk.norm2.weight, blk.ffn.up.weight.detach()[rank * fl:(rank + 1) * fl],
                                  blk.ffn.down.weight.detach()[:, rank * fl:(rank + 1) * fl], cfg.rms_eps, cfg.tau)
            layers += [attn, ffn]
        self.layers = nn.ModuleList(layers)

    def replicated_parameters(self) -> List[nn.Parameter]:
        """Parameters every rank holds in full and trains on its own tokens only (their gradients need a sum over ranks)."""
        out = list(self.embed.parameters()) + list(self.norm_f.parameters())
        if self.lm_head.weight is not self.embed.weight:
            out += list(self.lm_head.parameters())
        return out + [layer.norm_weight for layer in self.layers]

    def forward(self, tokens: torch.Tensor, labels: Optional[torch.Tensor] = None):
        """``tokens``: the FULL ``[B, S]`` batch on every rank.  Returns this rank's logits ``[n, vocab]`` (its slice of the
        flattened tokens) and, with ``labels``, its share of the mean next-token cross entropy."""
        from ..activation_based import functional
        functional.reset_net(self)
        n = self.ws.tokens_per_rank
        lo = self.rank * n
        flat = tokens.reshape(-1)
        x = self.embed(flat[lo:lo + n])                                       # [n, d]
        h = x.unsqueeze(0).expand(self.cfg.T, n, x.shape[-1])
        for layer in self.layers:
            h = layer(h)
        hidden = h.float().mean(0)
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=h.is_cuda):
            logits = self.lm_head(F.rms_norm(hidden, (hidden.shape[-1],), self.norm_f.weight.float(), self.norm_f.eps))
        if labels is None:
            return logits
        S = self.seq_len
        pos = torch.arange(lo, lo + n, device=tokens.device)
        has_next = (pos % S) != (S - 1)
        target = labels.reshape(-1)[(pos + 1).clamp(max=labels.numel() - 1)]
        per_token = F.cross_entropy(logits.float(), target, reduction="none")
        loss = (per_token * has_next).sum() / (self.batch * (S - 1))
        return logits, loss

    def check(self) -> None:
        self.ws.check()
