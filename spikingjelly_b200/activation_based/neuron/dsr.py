"""Import path of the reference's ``spikingjelly/activation_based/neuron/dsr.py``: the names below live in the ``neuron`` package here."""
from . import DSRIFNode, DSRLIFNode  # noqa: F401

__all__ = ['DSRIFNode', 'DSRLIFNode']
