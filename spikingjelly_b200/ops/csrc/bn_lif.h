// Host entry points shared between the BatchNorm-fused kernels.
#pragma once
#include <cuda_runtime.h>

namespace sjb200 {

// Adds the per-block partial sums [nblk][2][C] (sum g, sum g*y) in a fixed order and writes the BatchNorm
// parameter gradients and the coefficients (A, B, D) of the closed-form input gradient dy = A g + B y + D.
void launch_bn_finalize_backward(const float* partial, int nblk, int C, double count, int training, const float* gamma,
                                 const float* mean, const float* invstd, float* grad_gamma, float* grad_beta, float* coefA,
                                 float* coefB, float* coefD, cudaStream_t stream);

}  // namespace sjb200
