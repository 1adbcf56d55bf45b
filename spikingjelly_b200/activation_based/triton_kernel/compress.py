"""``bit_spike_compress`` / ``bit_spike_decompress`` under the reference's module path (``triton_kernel/compress.py:115-230``); the
implementation is the native bit-packing kernel (``ops/csrc/bitpack.cu``)."""
import torch

from ...ops import bitpack as _bitpack
from ...ops.bitpack import bit_spike_compress

__all__ = ["bit_spike_compress", "bit_spike_decompress"]


def bit_spike_decompress(s_seq_compressed: torch.Tensor, shape, dtype: torch.dtype = torch.bool) -> torch.Tensor:
    """The spikes packed by :func:`bit_spike_compress`, in ``shape``; ``dtype`` chooses what 0 / 1 are written as."""
    return _bitpack.bit_spike_decompress(s_seq_compressed, shape, dtype)
