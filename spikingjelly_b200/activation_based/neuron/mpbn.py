"""Import path of the reference's ``spikingjelly/activation_based/neuron/mpbn.py``: the names below live in the ``neuron`` package here."""
from . import MPBNBaseNode, MPBNLIFNode  # noqa: F401

__all__ = ['MPBNBaseNode', 'MPBNLIFNode']
