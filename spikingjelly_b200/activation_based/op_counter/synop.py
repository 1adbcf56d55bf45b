"""Import path of the reference's ``spikingjelly/activation_based/op_counter/synop.py``: the names below live in the ``op_counter`` package here."""
from . import SynOpCounter  # noqa: F401

__all__ = ['SynOpCounter']
