"""Import path of the reference's ``spikingjelly/activation_based/neuron/spikezip.py``: the names below live in the ``neuron`` package here."""
from . import STBIFNeuron  # noqa: F401

__all__ = ['STBIFNeuron']
