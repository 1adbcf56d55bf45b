"""Import path of the reference's ``spikingjelly/activation_based/neuron/inter_layer_connection.py``: the names below live in the ``neuron`` package here."""
from . import ILCBaseNode, ILCIFNode, ILCLIFNode, ILCCUBALIFNode  # noqa: F401

__all__ = ['ILCBaseNode', 'ILCIFNode', 'ILCLIFNode', 'ILCCUBALIFNode']
