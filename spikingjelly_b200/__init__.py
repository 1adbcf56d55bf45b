"""spikingjelly_b200 — a Blackwell (sm_100a) native spiking-neural-network framework.

The public Python surface mirrors SpikingJelly's ``spikingjelly.activation_based``
package (neurons, layers, surrogates, functional helpers, memopt, precision,
ann2snn, distributed) so that user code can switch by changing one import::

    from spikingjelly_b200.activation_based import neuron, layer, functional, surrogate

Hot paths run in hand-written CUDA kernels from :mod:`spikingjelly_b200.ops`.
"""

__version__ = "0.1.0"
__all__ = ["__version__"]
