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

// Delayed scaling in one pass.  `amax3` holds three slots used in rotation by successive calls on the same tensor role:
// call k scales with the maximum recorded by call k - 1 (slot (k + 2) % 3), records its own maximum in slot k % 3 and
// clears slot (k + 1) % 3 for the call after it, so no separate reduction or bookkeeping kernel runs.  Values beyond the
// previous maximum saturate at the format's largest number.
template <typename T, typename F8>
__global__ void __launch_bounds__(kThreads)
quantize_delayed_kernel(const T* __restrict__ x, long long n, float* __restrict__ amax3, int slot, float fmax, F8* __restrict__ q,
                        float* __restrict__ inv_scale) {
    constexpr int V = 16 / sizeof(T);
    const float a = amax3[(slot + 2) % 3];
    const float scale = a > 0.0f ? fmax / a : 1.0f;
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        *inv_scale = 1.0f / scale;
        amax3[(slot + 1) % 3] = 0.0f;
    }
    float m = 0.0f;
    const long long nv = n / V;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += (long long)gridDim.x * blockDim.x) {
        float v[V];
        load_vec_stream<T, V>(x + i * V, v);
        Pack<F8, V> out;
#pragma unroll
        for (int j = 0; j < V; ++j) {
            m = fmaxf(m, fabsf(v[j]));
            out.e[j] = F8(fminf(fmaxf(v[j] * scale, -fmax), fmax));
        }
        *reinterpret_cast<Pack<F8, V>*>(q + i * V) = out;
    }
    if (blockIdx.x == 0) {
        for (long long i = nv * V + threadIdx.x; i < n; i += blockDim.x) {
            const float v = to_f32<T>(x[i]);
            m = fmaxf(m, fabsf(v));
            q[i] = F8(fminf(fmaxf(v * scale, -fmax), fmax));
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    __shared__ float s[kThreads / 32];
    if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < kThreads / 32; ++w) m = fmaxf(m, s[w]);
        atomicMax(reinterpret_cast<unsigned int*>(amax3 + slot % 3), __float_as_uint(m));
    }
}

// Quantise a 16-bit matrix x [R, C] (R % 64 == 0, C % 128 == 0) and write both q [R, C] and its transpose qt [C, R] in one
// pass: the three products of a linear layer (forward, data gradient, weight gradient) contract over different axes,
// and the 8-bit tensor-core path wants the contraction axis contiguous in both operands.  One block moves a 64 x 128
// tile: 16-byte loads along the rows, the fp8 bytes staged in shared memory, 16-byte stores along the columns.
// `amax_in` gives the scale; with `amax_out` the tile maxima are accumulated there (delayed scaling) and `clear`
// (if given) is zeroed for the call after the next.
constexpr int kTileR = 64, kTileC = 128, kTilePitch = kTileC + 4;
template <typename T, typename F8>
__global__ void __launch_bounds__(kThreads)
quantize_transpose_kernel(const T* __restrict__ x, int R, int C, const float* __restrict__ amax_in, float* __restrict__ amax_out,
                          float* __restrict__ clear, float fmax, F8* __restrict__ q, F8* __restrict__ qt, float* __restrict__ inv_scale) {
    __shared__ __align__(16) unsigned char tile[kTileR * kTilePitch];
    __shared__ float red[kThreads / 32];
    const float a = *amax_in;
    const float scale = a > 0.0f ? fmax / a : 1.0f;
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        *inv_scale = 1.0f / scale;
        if (clear != nullptr) *clear = 0.0f;
    }
    const int tiles_c = C / kTileC, tiles = (R / kTileR) * tiles_c;
    const int cg = threadIdx.x & 15, r_in = threadIdx.x >> 4;
    float m = 0.0f;
    for (int t = blockIdx.x; t < tiles; t += gridDim.x) {
        const int r0 = (t / tiles_c) * kTileR, c0 = (t % tiles_c) * kTileC;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = r_in + 16 * i;
            float v[8];
            load_vec_stream<T, 8>(x + (size_t)(r0 + r) * C + c0 + cg * 8, v);
            Pack<F8, 8> out;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                m = fmaxf(m, fabsf(v[j]));
                out.e[j] = F8(fminf(fmaxf(v[j] * scale, -fmax), fmax));
            }
            *reinterpret_cast<Pack<F8, 8>*>(q + (size_t)(r0 + r) * C + c0 + cg * 8) = out;
            const uint2 w = *reinterpret_cast<const uint2*>(&out);
            uint32_t* dst = reinterpret_cast<uint32_t*>(tile + r * kTilePitch + cg * 8);
            dst[0] = w.x;
            dst[1] = w.y;
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int idx = threadIdx.x + kThreads * i;          // 128 columns x 4 row groups of 16
            const int c = idx >> 2, rg = idx & 3;
            uint32_t w[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const unsigned char* src = tile + (rg * 16 + k * 4) * kTilePitch + c;
                w[k] = (uint32_t)src[0] | ((uint32_t)src[kTilePitch] << 8) | ((uint32_t)src[2 * kTilePitch] << 16) |
                       ((uint32_t)src[3 * kTilePitch] << 24);
            }
            *reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(qt) + (size_t)(c0 + c) * R + r0 + rg * 16) = make_uint4(w[0], w[1], w[2], w[3]);
        }
        __syncthreads();
    }
    if (amax_out != nullptr) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int w = 1; w < kThreads / 32; ++w) m = fmaxf(m, red[w]);
            atomicMax(reinterpret_cast<unsigned int*>(amax_out), __float_as_uint(m));
        }
    }
}

}  // namespace

// (q [R, C], qt [C, R], inv_scale) of a 16-bit matrix in one pass over it.  Without `amax3` the scale comes from the
// tensor's own maximum (one extra read pass); with it, from the previous call on the same role (see fp8_quantize_delayed).
std::tuple<at::Tensor, at::Tensor, at::Tensor> fp8_quantize_transpose(const at::Tensor& x, const c10::optional<at::Tensor>& amax3,
                                                                      int64_t slot, bool e5m2) {
    TORCH_CHECK(x.is_cuda() && x.dim() == 2 && (x.scalar_type() == at::kBFloat16 || x.scalar_type() == at::kHalf),
                "fp8_quantize_transpose: 2-D bf16 / fp16 CUDA matrix required");
    const c10::cuda::CUDAGuard guard(x.device());
    at::Tensor xc = x.contiguous();
    const int64_t R = xc.size(0), C = xc.size(1);
    TORCH_CHECK(R % kTileR == 0 && C % kTileC == 0 && R > 0 && C > 0 && R < (1ll << 31) && C < (1ll << 31),
                "fp8_quantize_transpose: rows must be a multiple of 64 and columns of 128, got [", R, ", ", C, "]");
    TORCH_CHECK(reinterpret_cast<uintptr_t>(xc.data_ptr()) % 16 == 0, "fp8_quantize_transpose: input must be 16-byte aligned");
    const bool delayed = amax3.has_value() && amax3->defined();
    if (delayed)
        TORCH_CHECK(amax3->is_cuda() && amax3->scalar_type() == at::kFloat && amax3->numel() == 3 && amax3->is_contiguous() && slot >= 0,
                    "fp8_quantize_transpose: the state must be fp32[3] on the device and the slot non-negative");
    const auto f8 = e5m2 ? at::kFloat8_e5m2 : at::kFloat8_e4m3fn;
    at::Tensor q = at::empty({R, C}, xc.options().dtype(f8));
    at::Tensor qt = at::empty({C, R}, xc.options().dtype(f8));
    at::Tensor inv = at::empty({1}, xc.options().dtype(at::kFloat));
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    const float fmax = e5m2 ? 57344.0f : 448.0f;
    const long long n = xc.numel();
    at::Tensor own;
    const float* amax_in;
    float *amax_out = nullptr, *clear = nullptr;
    if (delayed) {
        float* s3 = amax3->data_ptr<float>();
        const int sl = (int)(slot % 3);
        amax_in = s3 + (sl + 2) % 3; amax_out = s3 + sl; clear = s3 + (sl + 1) % 3;
    } else {
        own = at::zeros({1}, xc.options().dtype(at::kFloat));
        amax_in = own.data_ptr<float>();
    }
    const int tiles = (int)((R / kTileR) * (C / kTileC));
    const unsigned grid = (unsigned)std::min(tiles, sms * 6);
    auto run = [&](auto tag) {
        using T = decltype(tag);
        const T* xp = reinterpret_cast<const T*>(xc.data_ptr());
        if (!delayed) {
            const unsigned g1 = (unsigned)std::max<long long>(1, std::min<long long>((n / 8 + kThreads - 1) / kThreads, (long long)sms * 8));
            absmax_kernel<T><<<g1, kThreads, 0, st>>>(xp, n, reinterpret_cast<unsigned int*>(own.data_ptr<float>()));
        }
        if (e5m2) quantize_transpose_kernel<T, __nv_fp8_e5m2><<<grid, kThreads, 0, st>>>(xp, (int)R, (int)C, amax_in, amax_out, clear, fmax,
                reinterpret_cast<__nv_fp8_e5m2*>(q.data_ptr()), reinterpret_cast<__nv_fp8_e5m2*>(qt.data_ptr()), inv.data_ptr<float>());
        else quantize_transpose_kernel<T, __nv_fp8_e4m3><<<grid, kThreads, 0, st>>>(xp, (int)R, (int)C, amax_in, amax_out, clear, fmax,
                reinterpret_cast<__nv_fp8_e4m3*>(q.data_ptr()), reinterpret_cast<__nv_fp8_e4m3*>(qt.data_ptr()), inv.data_ptr<float>());
    };
    if (xc.scalar_type() == at::kHalf) run(__half{}); else run(__nv_bfloat16{});
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return {q, qt, inv};
}

// One-pass quantisation with the scale of the previous call on the same tensor role (see quantize_delayed_kernel).
// amax3: fp32[3] state of the role; slot: the role's call counter (any non-negative integer; only slot % 3 matters).
std::tuple<at::Tensor, at::Tensor> fp8_quantize_delayed(const at::Tensor& x, at::Tensor amax3, int64_t slot, bool e5m2) {
    TORCH_CHECK(x.is_cuda() && amax3.is_cuda() && amax3.scalar_type() == at::kFloat && amax3.numel() == 3 && amax3.is_contiguous(),
                "fp8_quantize_delayed: CUDA input and an fp32[3] state tensor required");
    TORCH_CHECK(slot >= 0, "fp8_quantize_delayed: negative slot");
    const c10::cuda::CUDAGuard guard(x.device());
    at::Tensor xc = x.contiguous();
    TORCH_CHECK(reinterpret_cast<uintptr_t>(xc.data_ptr()) % 16 == 0, "fp8_quantize_delayed: input must be 16-byte aligned");
    const long long n = xc.numel();
    at::Tensor q = at::empty(xc.sizes(), xc.options().dtype(e5m2 ? at::kFloat8_e5m2 : at::kFloat8_e4m3fn));
    at::Tensor inv = at::empty({1}, xc.options().dtype(at::kFloat));
    if (n == 0) { inv.fill_(1.0); return {q, inv}; }
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    const float fmax = e5m2 ? 57344.0f : 448.0f;
    const int sl = (int)(slot % 3);
    auto run = [&](auto tag) {
        using T = decltype(tag);
        constexpr int V = 16 / sizeof(T);
        const unsigned grid = (unsigned)std::max<long long>(1, std::min<long long>((n / V + kThreads - 1) / kThreads, (long long)sms * 8));
        const T* xp = reinterpret_cast<const T*>(xc.data_ptr());
        if (e5m2) quantize_delayed_kernel<T, __nv_fp8_e5m2><<<grid, kThreads, 0, st>>>(xp, n, amax3.data_ptr<float>(), sl, fmax,
                                                                                    reinterpret_cast<__nv_fp8_e5m2*>(q.data_ptr()), inv.data_ptr<float>());
        else quantize_delayed_kernel<T, __nv_fp8_e4m3><<<grid, kThreads, 0, st>>>(xp, n, amax3.data_ptr<float>(), sl, fmax,
                                                                               reinterpret_cast<__nv_fp8_e4m3*>(q.data_ptr()), inv.data_ptr<float>());
    };
    switch (xc.scalar_type()) {
    case at::kFloat: run(float{}); break;
    case at::kHalf: run(__half{}); break;
    case at::kBFloat16: run(__nv_bfloat16{}); break;
    default: TORCH_CHECK(false, "fp8_quantize_delayed: fp32 / fp16 / bf16 input required, got ", xc.scalar_type());
    }
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return {q, inv};
}

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

TORCH_LIBRARY_FRAGMENT(sjb200, m) {
    m.def("fp8_quantize(Tensor x, bool e5m2) -> (Tensor, Tensor)");
    m.def("fp8_quantize_delayed(Tensor x, Tensor(a!) amax3, int slot, bool e5m2) -> (Tensor, Tensor)");
    m.def("fp8_quantize_transpose(Tensor x, Tensor(a!)? amax3, int slot, bool e5m2) -> (Tensor, Tensor, Tensor)");
}
TORCH_LIBRARY_IMPL(sjb200, CUDA, m) {
    m.impl("fp8_quantize", &sjb200::fp8_quantize);
    m.impl("fp8_quantize_delayed", &sjb200::fp8_quantize_delayed);
    m.impl("fp8_quantize_transpose", &sjb200::fp8_quantize_transpose);
}
