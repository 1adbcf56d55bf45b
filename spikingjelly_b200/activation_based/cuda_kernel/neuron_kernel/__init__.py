"""Import path of the reference's ``cuda_kernel/neuron_kernel`` (CuPy kernels for built-in and custom neurons).

Two layers, as there:

* functional entry points (``multi_step.integrate_and_fire.if_multi_step``, ``lif_multi_step``, ``plif_multi_step``, ``qif_multi_step``,
  ``eif_multi_step``, ``izhikevich_multi_step``, ``single_step.if_step``, ``lif_step``): these run the native scan kernels of
  this package (``ops/csrc/neuron_scan.cu``), the path ``backend="cupy"`` selects in the neuron modules;
* the extension classes for *custom* neurons (``multi_step.base.NeuronFPTTKernel`` / ``NeuronBPTTKernel`` / ``NeuronATGFBase``
  and the IF / LIF / PLIF kernels written with them): a kernel is assembled from code fragments - the user overrides
  ``neuronal_charge`` and the two gradient fragments - compiled by ``nvcc`` for sm_100a through ``auto_cuda`` and launched on
  PyTorch tensors.  They work on ``float`` tensors; 16-bit tensors take the native scan path.
"""
from . import multi_step, single_step  # noqa: F401
