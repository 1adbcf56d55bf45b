"""Reference import path ``op_counter.spikesim.counter``."""
from ._impl import SpikeSimCounter  # noqa: F401

__all__ = ['SpikeSimCounter']
