// Neuron scan kernels instantiated for __half storage.
#include "neuron_scan_launch.cuh"

namespace sjb200 {
SJ_SCAN_INSTANTIATE(__half)
}  // namespace sjb200
