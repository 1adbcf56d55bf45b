"""Import path of the reference's ``spikingjelly/activation_based/op_counter/neuromc/base_counter.py``: the names below live in the ``neuromc`` package here."""
from . import NeuroMCBaseCounter  # noqa: F401

__all__ = ['NeuroMCBaseCounter']
