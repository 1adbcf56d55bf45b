"""Import path of the reference's ``spikingjelly/activation_based/neuron/adapt.py``: the names below live in the ``neuron`` package here."""
from . import AdaptBaseNode, IzhikevichNode  # noqa: F401

__all__ = ['AdaptBaseNode', 'IzhikevichNode']
