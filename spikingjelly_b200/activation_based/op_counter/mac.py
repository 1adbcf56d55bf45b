"""Import path of the reference's ``spikingjelly/activation_based/op_counter/mac.py``: the names below live in the ``op_counter`` package here."""
from . import MACCounter  # noqa: F401

__all__ = ['MACCounter']
