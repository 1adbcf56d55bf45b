"""Import path of the reference's ``spikingjelly/activation_based/neuron/online_learning.py``: the names below live in the ``neuron`` package here."""
from . import OTTTLIFNode, SLTTLIFNode  # noqa: F401

__all__ = ['OTTTLIFNode', 'SLTTLIFNode']
