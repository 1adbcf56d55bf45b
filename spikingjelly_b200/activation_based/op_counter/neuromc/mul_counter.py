"""Import path of the reference's ``spikingjelly/activation_based/op_counter/neuromc/mul_counter.py``: the names below live in the ``neuromc`` package here."""
from . import NeuroMCMulCounter  # noqa: F401

__all__ = ['NeuroMCMulCounter']
