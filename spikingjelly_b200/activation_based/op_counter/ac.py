"""Import path of the reference's ``spikingjelly/activation_based/op_counter/ac.py``: the names below live in the ``op_counter`` package here."""
from . import ACCounter  # noqa: F401

__all__ = ['ACCounter']
