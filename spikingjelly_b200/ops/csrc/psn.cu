// Parallel spiking neuron (PSN family): H = W X + b over the time axis, S = (H >= 0), in one pass.
//
//   forward : reads X [T, N], writes S [T, N].  H never reaches memory: nothing but X is kept for backward.
//   backward: reads X and dS, recomputes H in registers, writes dX = W^T dH and dH = dS * g'(H); the tiny products
//             dW = dH X^T and db = sum_n dH are taken from dH by the caller.
//
// One thread owns V consecutive columns and the whole time axis of them: T x V inputs in registers, the T x T weight
// matrix and the bias in shared memory (broadcast reads).  Masked and sliding variants pass their effective matrix.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <torch/library.h>

#include "common.cuh"
#include "surrogate.cuh"

namespace sjb200 {
namespace {

constexpr int kThreads = 128;

template <typename T, int TT, int V>
__global__ void __launch_bounds__(kThreads)
psn_forward_kernel(const T* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b, T* __restrict__ s, int steps, long long n) {
    __shared__ float sw[TT * TT + TT];
    for (int i = threadIdx.x; i < steps * steps; i += kThreads) sw[(i / steps) * TT + (i % steps)] = w[i];
    for (int i = threadIdx.x; i < steps; i += kThreads) sw[TT * TT + i] = b[i];
    __syncthreads();
    const long long col = ((long long)blockIdx.x * kThreads + threadIdx.x) * V;
    if (col >= n) return;
    float xs[TT][V];
#pragma unroll
    for (int t = 0; t < TT; ++t)
        if (t < steps) load_vec_stream<T, V>(x + (long long)t * n + col, xs[t]);
#pragma unroll
    for (int t = 0; t < TT; ++t) {
        if (t >= steps) break;
        float h[V];
#pragma unroll
        for (int v = 0; v < V; ++v) h[v] = sw[TT * TT + t];
#pragma unroll
        for (int k = 0; k < TT; ++k) {
            if (k < steps) {
                const float wk = sw[t * TT + k];
#pragma unroll
                for (int v = 0; v < V; ++v) h[v] = fmaf(wk, xs[k][v], h[v]);
            }
        }
#pragma unroll
        for (int v = 0; v < V; ++v) h[v] = h[v] >= 0.0f ? 1.0f : 0.0f;
        store_vec<T, V>(s + (long long)t * n + col, h);
    }
}

template <typename T, int TT, int V>
__global__ void __launch_bounds__(kThreads)
psn_backward_kernel(const T* __restrict__ x, const T* __restrict__ gs, const float* __restrict__ w, const float* __restrict__ b,
                    T* __restrict__ gx, T* __restrict__ gh_out, int steps, long long n, int sg, float p0, float p1) {
    __shared__ float sw[TT * TT + TT];
    for (int i = threadIdx.x; i < steps * steps; i += kThreads) sw[(i / steps) * TT + (i % steps)] = w[i];
    for (int i = threadIdx.x; i < steps; i += kThreads) sw[TT * TT + i] = b[i];
    __syncthreads();
    const long long col = ((long long)blockIdx.x * kThreads + threadIdx.x) * V;
    if (col >= n) return;
    float xs[TT][V], acc[TT][V];
#pragma unroll
    for (int t = 0; t < TT; ++t) {
        if (t < steps) load_vec_stream<T, V>(x + (long long)t * n + col, xs[t]);
#pragma unroll
        for (int v = 0; v < V; ++v) acc[t][v] = 0.0f;
    }
#pragma unroll
    for (int t = 0; t < TT; ++t) {
        if (t >= steps) break;
        float h[V], g[V];
#pragma unroll
        for (int v = 0; v < V; ++v) h[v] = sw[TT * TT + t];
#pragma unroll
        for (int k = 0; k < TT; ++k) {
            if (k < steps) {
                const float wk = sw[t * TT + k];
#pragma unroll
                for (int v = 0; v < V; ++v) h[v] = fmaf(wk, xs[k][v], h[v]);
            }
        }
        load_vec_stream<T, V>(gs + (long long)t * n + col, g);
#pragma unroll
        for (int v = 0; v < V; ++v) g[v] *= surrogate_grad(sg, h[v], p0, p1);
        store_vec<T, V>(gh_out + (long long)t * n + col, g);
#pragma unroll
        for (int k = 0; k < TT; ++k) {
            if (k < steps) {
                const float wk = sw[t * TT + k];
#pragma unroll
                for (int v = 0; v < V; ++v) acc[k][v] = fmaf(wk, g[v], acc[k][v]);
            }
        }
    }
#pragma unroll
    for (int k = 0; k < TT; ++k)
        if (k < steps) store_vec<T, V>(gx + (long long)k * n + col, acc[k]);
}

// Backward for T <= 8: a thread walks several column groups and keeps its share of dW (T x T) and db (T) in registers;
// the block adds the shares in shared memory and writes one partial [T*T + T] per block, summed by the caller in a fixed
// order (deterministic).  No dH tensor is written.
template <typename T, int TT, int V>
__global__ void __launch_bounds__(kThreads)
psn_backward_small_kernel(const T* __restrict__ x, const T* __restrict__ gs, const float* __restrict__ w, const float* __restrict__ b,
                          T* __restrict__ gx, float* __restrict__ partial, int steps, long long n, int sg, float p0, float p1) {
    __shared__ float sw[TT * TT + TT];
    __shared__ float red[TT * TT + TT];
    for (int i = threadIdx.x; i < TT * TT + TT; i += kThreads) { sw[i] = 0.0f; red[i] = 0.0f; }
    __syncthreads();
    for (int i = threadIdx.x; i < steps * steps; i += kThreads) sw[(i / steps) * TT + (i % steps)] = w[i];
    for (int i = threadIdx.x; i < steps; i += kThreads) sw[TT * TT + i] = b[i];
    __syncthreads();
    float gw[TT][TT], gb[TT];
#pragma unroll
    for (int t = 0; t < TT; ++t) {
        gb[t] = 0.0f;
#pragma unroll
        for (int k = 0; k < TT; ++k) gw[t][k] = 0.0f;
    }
    const long long groups = n / V;
    for (long long grp = (long long)blockIdx.x * kThreads + threadIdx.x; grp < groups; grp += (long long)gridDim.x * kThreads) {
        const long long col = grp * V;
        float xs[TT][V], acc[TT][V];
#pragma unroll
        for (int t = 0; t < TT; ++t) {
#pragma unroll
            for (int v = 0; v < V; ++v) { xs[t][v] = 0.0f; acc[t][v] = 0.0f; }
            if (t < steps) load_vec_stream<T, V>(x + (long long)t * n + col, xs[t]);
        }
#pragma unroll
        for (int t = 0; t < TT; ++t) {
            if (t >= steps) break;
            float h[V], g[V];
#pragma unroll
            for (int v = 0; v < V; ++v) h[v] = sw[TT * TT + t];
#pragma unroll
            for (int k = 0; k < TT; ++k) {
                const float wk = sw[t * TT + k];                 // zero beyond `steps`
#pragma unroll
                for (int v = 0; v < V; ++v) h[v] = fmaf(wk, xs[k][v], h[v]);
            }
            load_vec_stream<T, V>(gs + (long long)t * n + col, g);
#pragma unroll
            for (int v = 0; v < V; ++v) {
                g[v] *= surrogate_grad(sg, h[v], p0, p1);
                gb[t] += g[v];
            }
#pragma unroll
            for (int k = 0; k < TT; ++k) {
                const float wk = sw[t * TT + k];
#pragma unroll
                for (int v = 0; v < V; ++v) {
                    acc[k][v] = fmaf(wk, g[v], acc[k][v]);
                    gw[t][k] = fmaf(g[v], xs[k][v], gw[t][k]);
                }
            }
        }
#pragma unroll
        for (int k = 0; k < TT; ++k)
            if (k < steps) store_vec<T, V>(gx + (long long)k * n + col, acc[k]);
    }
#pragma unroll
    for (int t = 0; t < TT; ++t) {
#pragma unroll
        for (int k = 0; k < TT; ++k) {
            const float v = warp_sum(gw[t][k]);
            if ((threadIdx.x & 31) == 0) atomicAdd(&red[t * TT + k], v);
        }
        const float v = warp_sum(gb[t]);
        if ((threadIdx.x & 31) == 0) atomicAdd(&red[TT * TT + t], v);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < TT * TT + TT; i += kThreads) partial[(long long)blockIdx.x * (TT * TT + TT) + i] = red[i];
}

struct Shape { int steps; long long n; };

Shape check(const at::Tensor& x, const at::Tensor& w, const at::Tensor& b, const char* who) {
    TORCH_CHECK(x.is_cuda() && x.dim() >= 2 && x.is_contiguous(), who, ": contiguous CUDA sequence [T, ...] required");
    const int steps = (int)x.size(0);
    TORCH_CHECK(steps >= 1 && steps <= 32, who, ": 1 <= T <= 32 supported, got ", steps);
    TORCH_CHECK(w.is_cuda() && w.scalar_type() == at::kFloat && w.is_contiguous() && w.dim() == 2 && w.size(0) == steps && w.size(1) == steps,
                who, ": weight must be fp32 [T, T]");
    TORCH_CHECK(b.is_cuda() && b.scalar_type() == at::kFloat && b.is_contiguous() && b.numel() == steps, who, ": bias must be fp32 with T values");
    const long long n = x.numel() / steps;
    TORCH_CHECK(reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0, who, ": input must be 16-byte aligned");
    return {steps, n};
}

// columns per thread: whole 16-byte accesses where the register budget allows (T x V inputs, twice that in backward)
template <typename T> constexpr int vec_for(int tt, bool backward) {
    const int full = 16 / (int)sizeof(T);
    const int budget = backward ? 64 : 128;
    int v = full;
    while (v > 1 && tt * v > budget) v /= 2;
    return v;
}

template <typename T, int TT, bool BWD, typename F>
void launch(long long n, F&& f) {
    constexpr int V = vec_for<T>(TT, BWD);
    TORCH_CHECK(n % V == 0, "psn: the number of neurons must be a multiple of ", V, " for this dtype and T");
    const unsigned grid = (unsigned)((n / V + kThreads - 1) / kThreads);
    f(std::integral_constant<int, V>{}, grid);
}

template <typename T, bool BWD, typename F>
void by_steps(int steps, long long n, F&& f) {
    if (steps <= 4) launch<T, 4, BWD>(n, [&](auto v, unsigned g) { f(std::integral_constant<int, 4>{}, v, g); });
    else if (steps <= 8) launch<T, 8, BWD>(n, [&](auto v, unsigned g) { f(std::integral_constant<int, 8>{}, v, g); });
    else if (steps <= 16) launch<T, 16, BWD>(n, [&](auto v, unsigned g) { f(std::integral_constant<int, 16>{}, v, g); });
    else launch<T, 32, BWD>(n, [&](auto v, unsigned g) { f(std::integral_constant<int, 32>{}, v, g); });
}

template <typename F>
void by_dtype(at::ScalarType t, F&& f) {
    switch (t) {
    case at::kFloat: f(float{}); break;
    case at::kHalf: f(__half{}); break;
    case at::kBFloat16: f(__nv_bfloat16{}); break;
    default: TORCH_CHECK(false, "psn: fp32 / fp16 / bf16 sequences supported, got ", t);
    }
}

}  // namespace

at::Tensor psn_forward(const at::Tensor& x, const at::Tensor& w, const at::Tensor& b) {
    const Shape sh = check(x, w, b, "psn_forward");
    const c10::cuda::CUDAGuard guard(x.device());
    at::Tensor s = at::empty_like(x);
    if (sh.n == 0) return s;
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    by_dtype(x.scalar_type(), [&](auto tag) {
        using T = decltype(tag);
        by_steps<T, false>(sh.steps, sh.n, [&](auto tt, auto v, unsigned grid) {
            psn_forward_kernel<T, decltype(tt)::value, decltype(v)::value><<<grid, kThreads, 0, st>>>(
                reinterpret_cast<const T*>(x.data_ptr()), w.data_ptr<float>(), b.data_ptr<float>(), reinterpret_cast<T*>(s.data_ptr()), sh.steps, sh.n);
        });
    });
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return s;
}

// returns (dX, dH); dW = dH X^T and db = sum over neurons of dH are left to the caller
std::tuple<at::Tensor, at::Tensor> psn_backward(const at::Tensor& x, const at::Tensor& grad_s, const at::Tensor& w, const at::Tensor& b,
                                                int64_t surrogate_id, double p0, double p1) {
    const Shape sh = check(x, w, b, "psn_backward");
    TORCH_CHECK(grad_s.is_cuda() && grad_s.is_contiguous() && grad_s.sizes() == x.sizes() && grad_s.scalar_type() == x.scalar_type(),
                "psn_backward: the spike gradient must match the input in shape and dtype");
    const c10::cuda::CUDAGuard guard(x.device());
    at::Tensor gx = at::empty_like(x), gh = at::empty_like(x);
    if (sh.n == 0) return {gx, gh};
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    by_dtype(x.scalar_type(), [&](auto tag) {
        using T = decltype(tag);
        by_steps<T, true>(sh.steps, sh.n, [&](auto tt, auto v, unsigned grid) {
            psn_backward_kernel<T, decltype(tt)::value, decltype(v)::value><<<grid, kThreads, 0, st>>>(
                reinterpret_cast<const T*>(x.data_ptr()), reinterpret_cast<const T*>(grad_s.data_ptr()), w.data_ptr<float>(), b.data_ptr<float>(),
                reinterpret_cast<T*>(gx.data_ptr()), reinterpret_cast<T*>(gh.data_ptr()), sh.steps, sh.n, (int)surrogate_id, (float)p0, (float)p1);
        });
    });
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return {gx, gh};
}

// T <= 8: returns (dX, dW [T, T] fp32, db [T] fp32) without writing dH.
std::tuple<at::Tensor, at::Tensor, at::Tensor> psn_backward_small(const at::Tensor& x, const at::Tensor& grad_s, const at::Tensor& w,
                                                                  const at::Tensor& b, int64_t surrogate_id, double p0, double p1) {
    const Shape sh = check(x, w, b, "psn_backward_small");
    TORCH_CHECK(sh.steps <= 8, "psn_backward_small: T <= 8 required");
    TORCH_CHECK(grad_s.is_cuda() && grad_s.is_contiguous() && grad_s.sizes() == x.sizes() && grad_s.scalar_type() == x.scalar_type(),
                "psn_backward_small: the spike gradient must match the input in shape and dtype");
    const c10::cuda::CUDAGuard guard(x.device());
    at::Tensor gx = at::empty_like(x);
    const int TT = sh.steps <= 4 ? 4 : 8, slot = TT * TT + TT;
    const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    at::Tensor partial;
    by_dtype(x.scalar_type(), [&](auto tag) {
        using T = decltype(tag);
        auto run = [&](auto tt) {
            constexpr int kTT = decltype(tt)::value;
            constexpr int V = (16 / (int)sizeof(T)) > 4 ? 4 : (16 / (int)sizeof(T));
            TORCH_CHECK(sh.n % V == 0, "psn: the number of neurons must be a multiple of ", V);
            const long long groups = sh.n / V;
            const unsigned grid = (unsigned)std::max<long long>(1, std::min<long long>((groups + kThreads - 1) / kThreads, (long long)sms * 6));
            partial = at::empty({(long long)grid, slot}, x.options().dtype(at::kFloat));
            psn_backward_small_kernel<T, kTT, V><<<grid, kThreads, 0, st>>>(
                reinterpret_cast<const T*>(x.data_ptr()), reinterpret_cast<const T*>(grad_s.data_ptr()), w.data_ptr<float>(), b.data_ptr<float>(),
                reinterpret_cast<T*>(gx.data_ptr()), partial.data_ptr<float>(), sh.steps, sh.n, (int)surrogate_id, (float)p0, (float)p1);
        };
        if (TT == 4) run(std::integral_constant<int, 4>{}); else run(std::integral_constant<int, 8>{});
    });
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    at::Tensor total = partial.sum(0);
    at::Tensor gw = total.narrow(0, 0, TT * TT).view({TT, TT}).narrow(0, 0, sh.steps).narrow(1, 0, sh.steps).contiguous();
    at::Tensor gb = total.narrow(0, TT * TT, sh.steps).contiguous();
    return {gx, gw, gb};
}

}  // namespace sjb200

TORCH_LIBRARY_FRAGMENT(sjb200, m) {
    m.def("psn_forward(Tensor x, Tensor w, Tensor b) -> Tensor");
    m.def("psn_backward(Tensor x, Tensor grad_s, Tensor w, Tensor b, int surrogate_id, float p0, float p1) -> (Tensor, Tensor)");
    m.def("psn_backward_small(Tensor x, Tensor grad_s, Tensor w, Tensor b, int surrogate_id, float p0, float p1) -> (Tensor, Tensor, Tensor)");
}
TORCH_LIBRARY_IMPL(sjb200, CUDA, m) {
    m.impl("psn_forward", &sjb200::psn_forward);
    m.impl("psn_backward", &sjb200::psn_backward);
    m.impl("psn_backward_small", &sjb200::psn_backward_small);
}
