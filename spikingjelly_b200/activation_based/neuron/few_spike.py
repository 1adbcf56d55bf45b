"""Import path of the reference's ``spikingjelly/activation_based/neuron/few_spike.py``: the names below live in the ``neuron`` package here."""
from . import FewSpikeTable, FewSpikeNode, OutlierAwareThresholdNode, HGNode  # noqa: F401

__all__ = ['FewSpikeTable', 'FewSpikeNode', 'OutlierAwareThresholdNode', 'HGNode']

from typing import Sequence, Union  # noqa: E402

import torch  # noqa: E402

#: what the few-spike neuron accepts for its per-step coefficient vectors
TensorLike1D = Union[torch.Tensor, Sequence[float]]
