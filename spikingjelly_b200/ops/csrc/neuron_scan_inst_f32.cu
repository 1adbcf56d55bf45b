// Neuron scan kernels instantiated for float storage.
#include "neuron_scan_launch.cuh"

namespace sjb200 {
SJ_SCAN_INSTANTIATE(float)
}  // namespace sjb200
