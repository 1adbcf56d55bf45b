"""Multi-step kernels and the custom-neuron extension classes (``cuda_kernel/neuron_kernel/multi_step/`` of the reference)."""
from . import base, eif, integrate_and_fire, izhikevich, lif, plif, qif  # noqa: F401
from .base import NeuronATGFBase, NeuronBPTTKernel, NeuronFPTTKernel
from .integrate_and_fire import IFNodeBPTTKernel, IFNodeFPTTKernel
from .lif import LIFNodeBPTTKernel, LIFNodeFPTTKernel
from .plif import ParametricLIFNodeBPTTKernel, ParametricLIFNodeFPTTKernel

__all__ = ["IFNodeBPTTKernel", "IFNodeFPTTKernel", "LIFNodeBPTTKernel", "LIFNodeFPTTKernel", "NeuronATGFBase", "NeuronBPTTKernel",
           "NeuronFPTTKernel", "ParametricLIFNodeBPTTKernel", "ParametricLIFNodeFPTTKernel"]
