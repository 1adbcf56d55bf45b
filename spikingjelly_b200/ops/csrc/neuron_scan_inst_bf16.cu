// Neuron scan kernels instantiated for __nv_bfloat16 storage.
#include "neuron_scan_launch.cuh"

namespace sjb200 {
SJ_SCAN_INSTANTIATE(__nv_bfloat16)
}  // namespace sjb200
