"""Import path of the reference's ``spikingjelly/activation_based/neuron/noisy.py``: the names below live in the ``neuron`` package here."""
from . import (  # noqa: F401
    powerlaw_psd_gaussian, NoisyBaseNode, NoisyCUBALIFNode, NoisyILCBaseNode, NoisyILCCUBALIFNode,
    NoisyNonSpikingBaseNode, NoisyNonSpikingIFNode)

__all__ = ['powerlaw_psd_gaussian', 'NoisyBaseNode', 'NoisyCUBALIFNode', 'NoisyILCBaseNode',
           'NoisyILCCUBALIFNode', 'NoisyNonSpikingBaseNode', 'NoisyNonSpikingIFNode']
