"""Spike tensors stored as booleans or as bits (``cuda_kernel/tensor_cache.py:96-333`` of the reference).

``float_spike_to_bool`` packs 8 spikes per byte (bit ``i`` of byte ``j`` = element ``8 j + i``) with the bit-packing kernel of
the native library on CUDA tensors and with integer arithmetic elsewhere; ``BoolTensorCache`` is the reference-counted store
that ``spike_op`` keeps its saved inputs in (``configure.save_bool_spike_level``: 0 = ``bool`` tensor, 1 = bits)."""
from __future__ import annotations

import threading
from typing import Tuple

import torch

from ... import configure
from ...ops import bitpack

__all__ = ["float_spike_to_bool", "bool_spike_to_float", "tensor_key", "BoolTensorCache", "BOOL_TENSOR_CACHE", "DataTypeConvertCUDACode"]


def float_spike_to_bool(spike: torch.Tensor) -> Tuple[torch.Tensor, torch.dtype, torch.Size, int]:
    """-> ``(packed uint8, dtype, shape, padding)``; ``padding`` = zero bits appended to fill the last byte."""
    if not spike.is_floating_point():
        raise NotImplementedError(spike.dtype)
    numel = spike.numel()
    padding = (8 - numel % 8) % 8
    return bitpack.bit_spike_compress(spike), spike.dtype, spike.shape, padding


def bool_spike_to_float(spike_b: torch.Tensor, s_dtype: torch.dtype, s_shape: torch.Size, s_padding: int = 0) -> torch.Tensor:
    return bitpack.bit_spike_decompress(spike_b, s_shape, s_dtype)


def tensor_key(x: torch.Tensor):
    x = x.flatten()
    return x.data_ptr(), x[-1].data_ptr(), x.numel()


class BoolTensorCache:
    """``store_bool(spike) -> key`` / ``get_float(key, shape)``; an entry stored k times is released by the k-th ``get_float``."""

    def __init__(self):
        self.cache = {}
        self.lock = threading.Lock()

    def store_bool(self, spike: torch.Tensor):
        tk = tensor_key(spike)
        with self.lock:
            entry = self.cache.get(tk)
            if entry is not None:
                self.cache[tk] = (entry[0], entry[1] + 1)
            elif configure.save_bool_spike_level == 0:
                self.cache[tk] = ((spike.bool(), spike.dtype), 1)
            elif configure.save_bool_spike_level == 1:
                self.cache[tk] = (float_spike_to_bool(spike), 1)
            else:
                raise NotImplementedError(configure.save_bool_spike_level)
        return tk

    def get_float(self, tk, spike_shape: torch.Size) -> torch.Tensor:
        with self.lock:
            payload, refs = self.cache[tk]
            if refs == 1:
                del self.cache[tk]
            else:
                self.cache[tk] = (payload, refs - 1)
        if len(payload) == 2:
            spike = payload[0].to(payload[1])
        else:
            spike = bool_spike_to_float(*payload)
        return spike.view(spike_shape)


BOOL_TENSOR_CACHE = BoolTensorCache()


class DataTypeConvertCUDACode:
    """Where the conversion kernels live.  The reference keeps four CuPy source strings under these attribute names
    (``float2bool``, ``half2bool``, ``bool2float``, ``bool2half``: 8 spikes <-> 1 byte); here the conversions are compiled
    kernels of the native library (32 spikes <-> one 32-bit word, any floating dtype), and each attribute names its entry point."""
    source_file = "spikingjelly_b200/ops/csrc/bitpack.cu"
    float2bool = half2bool = "torch.ops.sjb200.bit_pack"
    bool2float = bool2half = "torch.ops.sjb200.bit_unpack"
