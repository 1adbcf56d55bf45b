"""Bit packing of spike tensors (8 spikes per byte; bit ``i`` of byte ``j`` is element ``8 j + i``)."""
from __future__ import annotations

import torch

__all__ = ["bit_spike_compress", "bit_spike_decompress"]


def _pack_torch(flat_bool: torch.Tensor) -> torch.Tensor:
    n = flat_bool.numel()
    pad = (-n) % 8
    if pad:
        flat_bool = torch.cat([flat_bool, flat_bool.new_zeros(pad)])
    weights = torch.tensor([1, 2, 4, 8, 16, 32, 64, 128], dtype=torch.uint8, device=flat_bool.device)
    return (flat_bool.view(-1, 8).to(torch.uint8) * weights).sum(dim=1, dtype=torch.uint8)


def bit_spike_compress(s_seq: torch.Tensor) -> torch.Tensor:
    """``uint8[(numel + 7) // 8]`` holding ``s_seq != 0`` bit by bit."""
    if s_seq.is_cuda and s_seq.dtype in (torch.float32, torch.float16, torch.bfloat16):
        from . import counters, require
        require()
        counters.bump("bit_pack")
        return torch.ops.sjb200.bit_pack(s_seq)
    return _pack_torch((s_seq != 0).reshape(-1))


def bit_spike_decompress(packed: torch.Tensor, shape, dtype: torch.dtype = torch.bool) -> torch.Tensor:
    n = 1
    for s in shape:
        n *= int(s)
    if packed.is_cuda and dtype in (torch.float32, torch.float16, torch.bfloat16):
        from . import counters, require
        require()
        counters.bump("bit_unpack")
        return torch.ops.sjb200.bit_unpack(packed, n, dtype).reshape(shape)
    shifts = torch.arange(8, dtype=torch.uint8, device=packed.device)
    bits = ((packed.unsqueeze(1) >> shifts) & 1).reshape(-1)[:n]
    return bits.to(dtype).reshape(shape)
