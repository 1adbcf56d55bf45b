// Surrogate derivative table.  Ids match SURROGATES in activation_based/surrogate.py.
#pragma once
#include <cuda_runtime.h>

namespace sjb200 {

enum SurrogateId : int {
    SG_SIGMOID = 0, SG_ATAN = 1, SG_PIECEWISE_QUADRATIC = 2, SG_PIECEWISE_EXP = 3, SG_SOFT_SIGN = 4,
    SG_SUPER_SPIKE = 5, SG_ERF = 6, SG_NONZERO_SIGN_LOG_ABS = 7, SG_PIECEWISE_LEAKY_RELU = 8,
    SG_SQUAREWAVE = 9, SG_S2NN = 10, SG_Q_PSEUDO_SPIKE = 11, SG_LEAKY_K_RELU = 12,
    SG_FAKE_NUMERICAL = 13, SG_LOG_TAILED_RELU = 14, SG_DETERMINISTIC_PASS = 15, SG_RECT = 16,
};

// g'(x) for surrogate `id` with parameters (p0, p1).  `id` is uniform across the
// grid, so the switch costs one predictable branch.
__device__ __forceinline__ float surrogate_grad(int id, float x, float p0, float p1) {
    const float PI = 3.14159265358979323846f;
    switch (id) {
    case SG_SIGMOID: { float s = __fdividef(1.0f, 1.0f + __expf(-p0 * x)); return (1.0f - s) * s * p0; }
    case SG_ATAN: { float a = p0 * 0.5f; float ax = PI * a * x; return __fdividef(a, 1.0f + ax * ax); }
    case SG_PIECEWISE_QUADRATIC: { float xa = fabsf(x); return xa > (1.0f / p0) ? 0.0f : (-(p0 * p0) * xa + p0); }
    case SG_PIECEWISE_EXP: return p0 * 0.5f * expf(-p0 * fabsf(x));
    case SG_SOFT_SIGN: { float d = 1.0f / p0 + fabsf(x); return 1.0f / (2.0f * p0 * d * d); }
    case SG_SUPER_SPIKE: { float d = fabsf(x) + 1.0f; return p0 / (d * d); }
    case SG_ERF: { float ax = x * p0; return expf(-ax * ax) * (p0 * 0.5641895835477563f); }
    case SG_NONZERO_SIGN_LOG_ABS: return 1.0f / (1.0f / p0 + fabsf(x));
    case SG_PIECEWISE_LEAKY_RELU: return fabsf(x) < p0 ? 1.0f / (2.0f * p0) : p1;
    case SG_SQUAREWAVE: {
        float w = 2.0f * PI / p1, g = 0.0f; int n = (int)p0;
        for (int i = 1; i < n; ++i) g += cosf((2.0f * i - 1.0f) * w * x);
        return g * (4.0f / p1);
    }
    case SG_S2NN: {
        if (x < 0.0f) { float s = 1.0f / (1.0f + expf(-p0 * x)); return p0 * s * (1.0f - s); }
        return p1 / (x + 1.0f);
    }
    case SG_Q_PSEUDO_SPIKE: return powf(1.0f + 2.0f / (p0 - 1.0f) * fabsf(x), -p0);
    case SG_LEAKY_K_RELU: return x >= 0.0f ? p1 : p0;
    case SG_FAKE_NUMERICAL: return fminf((x >= 0.0f ? 1.0f : -1.0f) / x, p0);
    case SG_LOG_TAILED_RELU: return x <= 0.0f ? p0 : (x > 1.0f ? 1.0f / x : 1.0f);
    case SG_DETERMINISTIC_PASS: return 1.0f;
    case SG_RECT: return fabsf(x) < 0.5f / p0 ? p0 : 0.0f;
    default: return 0.0f;
    }
}

template <int ID>
__device__ __forceinline__ float surrogate_grad(float x, float p0, float p1) { return surrogate_grad(ID, x, p0, p1); }

// Out-of-line copy of the full table for the rarely used surrogates: one body per translation
// unit instead of one per unrolled call site (the inlined table dominated compile time and code size).
static __device__ __noinline__ float surrogate_grad_outlined(int id, float x, float p0, float p1) {
    return surrogate_grad(id, x, p0, p1);
}

// In-place g'(x) for V values.  The two surrogates used by every shipped model get
// branch-free bodies; the switch for the rest is taken once per call, not per element.
template <int V>
__device__ __forceinline__ void surrogate_grad_vec(int id, float (&x)[V], float p0, float p1) {
    if (id == SG_ATAN) {
        const float a = p0 * 0.5f, pa = 3.14159265358979323846f * a;
#pragma unroll
        for (int j = 0; j < V; ++j) { const float ax = pa * x[j]; x[j] = __fdividef(a, 1.0f + ax * ax); }
    } else if (id == SG_SIGMOID) {
#pragma unroll
        for (int j = 0; j < V; ++j) { const float s = __fdividef(1.0f, 1.0f + __expf(-p0 * x[j])); x[j] = (1.0f - s) * s * p0; }
    } else {
#pragma unroll
        for (int j = 0; j < V; ++j) x[j] = surrogate_grad_outlined(id, x[j], p0, p1);
    }
}

}  // namespace sjb200
