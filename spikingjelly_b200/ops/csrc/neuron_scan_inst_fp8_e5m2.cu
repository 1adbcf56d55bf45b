// Neuron scan kernels with fp8-e5m2 input storage (the wide-range 8-bit format): x_seq is read as one byte per element,
// spikes, states and every gradient are bf16.
#include <cuda_fp8.h>

#include "neuron_scan_launch.cuh"

namespace sjb200 {
SJ_SCAN_INSTANTIATE2(__nv_fp8_e5m2, __nv_bfloat16)
}  // namespace sjb200
