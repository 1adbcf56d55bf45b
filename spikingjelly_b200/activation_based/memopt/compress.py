"""Spike compressors for activation checkpointing: what is stored between forward and backward.

Parity: ``spikingjelly/activation_based/memopt/compress.py:57-457``.  ``BitSpikeCompressor`` uses
the native bit-pack kernel on CUDA (``ops/csrc/bitpack.cu``) and PyTorch ops elsewhere.
"""
from __future__ import annotations

import abc

import torch

from ...ops.bitpack import bit_spike_compress, bit_spike_decompress

__all__ = ["BaseSpikeCompressor", "NullSpikeCompressor", "BooleanSpikeCompressor", "Uint8SpikeCompressor",
           "BitSpikeCompressor", "SparseSpikeCompressor", "bit_spike_compress", "bit_spike_decompress"]


class BaseSpikeCompressor(abc.ABC):
    """``compress(x) -> stored tensor``; ``decompress(stored, shape) -> x`` (both without autograd).
    ``requires_strictly_binary``: the round trip is only lossless for inputs in {0, 1}."""
    requires_strictly_binary = False

    def __init__(self):
        self.s_seq_dtype = torch.float32

    @abc.abstractmethod
    def _compress(self, s_seq: torch.Tensor) -> torch.Tensor:
        ...

    @abc.abstractmethod
    def _decompress(self, s_seq: torch.Tensor, shape) -> torch.Tensor:
        ...

    def compress(self, s_seq: torch.Tensor) -> torch.Tensor:
        with torch.no_grad():
            return self._compress(s_seq)

    def decompress(self, s_seq: torch.Tensor, shape) -> torch.Tensor:
        with torch.no_grad():
            return self._decompress(s_seq, shape)


class NullSpikeCompressor(BaseSpikeCompressor):
    def _compress(self, s_seq):
        return s_seq

    def _decompress(self, s_seq, shape):
        return s_seq


class _CastCompressor(BaseSpikeCompressor):
    _store = torch.bool

    def _compress(self, s_seq):
        self.s_seq_dtype = s_seq.dtype
        return s_seq.to(dtype=self._store)

    def _decompress(self, s_seq, shape):
        return s_seq.to(dtype=self.s_seq_dtype).reshape(shape)


class BooleanSpikeCompressor(_CastCompressor):
    """One byte per spike."""
    requires_strictly_binary = True
    _store = torch.bool


class Uint8SpikeCompressor(_CastCompressor):
    """One byte per value; keeps small integer spike counts (0..255)."""
    _store = torch.uint8


class BitSpikeCompressor(BaseSpikeCompressor):
    """One bit per spike: 16x smaller than bf16, 32x smaller than fp32."""
    requires_strictly_binary = True

    def _compress(self, s_seq):
        self.s_seq_dtype = s_seq.dtype
        return bit_spike_compress(s_seq)

    def _decompress(self, s_seq, shape):
        dt = self.s_seq_dtype
        if s_seq.is_cuda and dt in (torch.float32, torch.float16, torch.bfloat16):
            return bit_spike_decompress(s_seq, shape, dt)
        return bit_spike_decompress(s_seq, shape, torch.bool).to(dtype=dt)


class SparseSpikeCompressor(BaseSpikeCompressor):
    """Stores the indices of the non-zero entries (pays off below ~3 % firing rate with int32)."""
    requires_strictly_binary = True

    def __init__(self, dtype=torch.int64):
        super().__init__()
        self.dtype = dtype

    def _compress(self, s_seq):
        self.s_seq_dtype = s_seq.dtype
        return torch.nonzero(s_seq.reshape(-1)).to(dtype=self.dtype)

    def _decompress(self, s_seq, shape):
        n = torch.Size(shape).numel()
        out = torch.zeros(n, dtype=self.s_seq_dtype, device=s_seq.device)
        return out.scatter_(0, s_seq.to(torch.int64).reshape(-1), 1).reshape(shape)
