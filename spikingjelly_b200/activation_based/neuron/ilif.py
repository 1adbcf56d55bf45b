"""Import path of the reference's ``spikingjelly/activation_based/neuron/ilif.py``: the names below live in the ``neuron`` package here."""
from . import ILIFNode  # noqa: F401

__all__ = ['ILIFNode']
