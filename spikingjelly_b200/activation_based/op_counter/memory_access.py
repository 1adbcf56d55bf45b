"""Import path of the reference's ``spikingjelly/activation_based/op_counter/memory_access.py``: the names below live in the ``op_counter`` package here."""
from . import MemoryAccessCounter  # noqa: F401

__all__ = ['MemoryAccessCounter']
