"""Import path of the reference's ``spikingjelly/activation_based/op_counter/flop.py``: the names below live in the ``op_counter`` package here."""
from . import FlopCounter  # noqa: F401

__all__ = ['FlopCounter']
