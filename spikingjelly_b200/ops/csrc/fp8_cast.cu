// Per-tensor dynamic fp8 quantisation: absolute maximum (one pass, order-independent atomic max)
// and scaled cast to e4m3 / e5m2 (one pass).  The scale never visits the host:
//     scale = fmax / amax  (1 when the tensor is all zero),  q = cast(x * scale),  inv_scale = 1 / scale.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_fp8.h>
#include <torch/library.h>

#include "common.cuh"

namespace sjb200 {
namespace {

constexpr int kThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kThreads)
absmax_kernel(const T* __restrict__ x, long long n, unsigned int* __restrict__ out_bits) {
    constexpr int V = 16 / sizeof(T);
    float m = 0.0f;
    const long long nv = n / V;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += (long long)gridDim.x * blockDim.x) {
        float v[V];
        load_vec_stream<T, V>(x + i * V, v);
#pragma unroll
        for (int j = 0; j < V; ++j) m = fmaxf(m, fabsf(v[j]));
    }
    if (blockIdx.x == 0) {
        for (long long i = nv * V + threadIdx.x; i < n; i += blockDim.x) m = fmaxf(m, fabsf(to_f32<T>(x[i])));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    __shared__ float s[kThreads / 32];
    if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < kThreads / 32; ++w) m = fmaxf(m, s[w]);
        atomicMax(out_bits, __float_as_uint(m));     // non-negative floats order like their bit patterns
    }
}

template <typename T, typename F8>
__global__ void __launch_bounds__(kThreads)
quantize_kernel(const T* __restrict__ x, long long n, const float* __restrict__ amax, float fmax, F8* __restrict__ q,
                float* __restrict__ inv_scale) {
    constexpr int V = 16 / sizeof(T);
    const float a = *amax;
    const float scale = a > 0.0f ? fmax / a : 1.0f;
    if (blockIdx.x == 0 && threadIdx.x == 0) *inv_scale = 1.0f / scale;
    const long long nv = n / V;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += (long long)gridDim.x * blockDim.x) {
        float v[V];
        load_vec_stream<T, V>(x + i * V, v);
        Pack<F8, V> out;
#pragma unroll
        for (int j = 0; j < V; ++j) out.e[j] = F8(fminf(fmaxf(v[j] * scale, -fmax), fmax));
        *reinterpret_cast<Pack<F8, V>*>(q + i * V) = out;
    }
    if (blockIdx.x == 0) {
        for (long long i = nv * V + threadIdx.x; i < n; i += blockDim.x)
            q[i] = F8(fminf(fmaxf(to_f32<T>(x[i]) * scale, -fmax), fmax));
    }
}

}  // namespace

// returns (q fp8 like x, inv_scale fp32[1]);  e5m2 == false: float8_e4m3fn (max 448), else float8_e5m2 (max 57344)
std::tuple<at::Tensor, at::Tensor> fp8_quantize(const at::Tensor& x, bool e5m2) {
    TORCH_CHECK(x.is_cuda(), "fp8_quantize: CUDA tensor required");
    const c10::cuda::CUDAGuard guard(x.device());
    at::Tensor xc = x.contiguous();
    TORCH_CHECK(reinterpret_cast<uintptr_t>(xc.data_ptr()) % 16 == 0, "fp8_quantize: input must be 16-byte aligned");
    const long long n = xc.numel();
    at::Tensor q = at::empty(xc.sizes(), xc.options().dtype(e5m2 ? at::kFloat8_e5m2 : at::kFloat8_e4m3fn));
    at::Tensor amax = at::zeros({1}, xc.options().dtype(at::kFloat));
    at::Tensor inv = at::empty({1}, xc.options().dtype(at::kFloat));
    if (n == 0) { inv.fill_(1.0); return {q, inv}; }
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    const float fmax = e5m2 ? 57344.0f : 448.0f;
    auto run = [&](auto tag) {
        using T = decltype(tag);
        constexpr int V = 16 / sizeof(T);
        const unsigned grid = (unsigned)std::max<long long>(1, std::min<long long>((n / V + kThreads - 1) / kThreads, (long long)sms * 8));
        const T* xp = reinterpret_cast<const T*>(xc.data_ptr());
        absmax_kernel<T><<<grid, kThreads, 0, st>>>(xp, n, reinterpret_cast<unsigned int*>(amax.data_ptr<float>()));
        if (e5m2) quantize_kernel<T, __nv_fp8_e5m2><<<grid, kThreads, 0, st>>>(xp, n, amax.data_ptr<float>(), fmax,
                                                                            reinterpret_cast<__nv_fp8_e5m2*>(q.data_ptr()), inv.data_ptr<float>());
        else quantize_kernel<T, __nv_fp8_e4m3><<<grid, kThreads, 0, st>>>(xp, n, amax.data_ptr<float>(), fmax,
                                                                       reinterpret_cast<__nv_fp8_e4m3*>(q.data_ptr()), inv.data_ptr<float>());
    };
    switch (xc.scalar_type()) {
    case at::kFloat: run(float{}); break;
    case at::kHalf: run(__half{}); break;
    case at::kBFloat16: run(__nv_bfloat16{}); break;
    default: TORCH_CHECK(false, "fp8_quantize: fp32 / fp16 / bf16 input required, got ", xc.scalar_type());
    }
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return {q, inv};
}

}  // namespace sjb200

TORCH_LIBRARY_FRAGMENT(sjb200, m) { m.def("fp8_quantize(Tensor x, bool e5m2) -> (Tensor, Tensor)"); }
TORCH_LIBRARY_IMPL(sjb200, CUDA, m) { m.impl("fp8_quantize", &sjb200::fp8_quantize); }
