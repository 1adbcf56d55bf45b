"""Legacy import path of :class:`GaussianTuning` (``spikingjelly/timing_based/orig_encoding.py``)."""
from .encoding import GaussianTuning  # noqa: F401
