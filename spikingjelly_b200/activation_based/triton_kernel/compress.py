"""``bit_spike_compress`` / ``bit_spike_decompress`` under the reference's module path (``triton_kernel/compress.py:115-200``); the
implementation is the native bit-packing kernel (``ops/csrc/bitpack.cu``)."""
from ...ops.bitpack import bit_spike_compress, bit_spike_decompress

__all__ = ["bit_spike_compress", "bit_spike_decompress"]
