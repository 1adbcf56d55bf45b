"""Import path of the reference's ``spikingjelly/activation_based/neuron/plif.py``: the names below live in the ``neuron`` package here."""
from . import ParametricLIFNode  # noqa: F401

__all__ = ['ParametricLIFNode']
