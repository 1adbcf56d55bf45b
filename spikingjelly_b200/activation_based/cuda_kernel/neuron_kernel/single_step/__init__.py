"""Single-step neuron kernels (``cuda_kernel/neuron_kernel/single_step/`` of the reference)."""
from . import base, integrate_and_fire, lif  # noqa: F401
from .base import NeuronBPKernel, NeuronFPKernel  # noqa: F401
