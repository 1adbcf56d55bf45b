// Bit packing of spike tensors: 8 spikes per byte (bit i of byte j is element 8 j + i).
// One thread packs 16 bytes' worth (128 elements, read as 128-bit vectors) — the kernel is a pure
// stream: read n * sizeof(T), write n / 8 bytes.  Unpacking is the mirror image.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "common.cuh"

namespace sjb200 {
namespace {

constexpr int kThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kThreads)
bit_pack_kernel(const T* __restrict__ x, uint8_t* __restrict__ out, long long n) {
    constexpr int V = 16 / sizeof(T);                  // elements per 128-bit load
    const long long byte0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * (V >= 8 ? V / 8 : 1);
    const long long e0 = byte0 * 8;
    if (e0 >= n) return;
    constexpr int ELEMS = V >= 8 ? V : 8;
    uint32_t bits = 0;
    if (e0 + ELEMS <= n && (reinterpret_cast<uintptr_t>(x + e0) % 16 == 0)) {
#pragma unroll
        for (int v = 0; v < ELEMS / V; ++v) {
            float f[V];
            load_vec_stream<T, V>(x + e0 + v * V, f);
#pragma unroll
            for (int j = 0; j < V; ++j) bits |= (f[j] != 0.0f ? 1u : 0u) << (v * V + j);
        }
    } else {
        for (int j = 0; j < ELEMS && e0 + j < n; ++j) bits |= (to_f32<T>(x[e0 + j]) != 0.0f ? 1u : 0u) << j;
    }
    const long long nbytes = (n + 7) / 8;
#pragma unroll
    for (int b = 0; b < ELEMS / 8; ++b)
        if (byte0 + b < nbytes) out[byte0 + b] = (uint8_t)((bits >> (8 * b)) & 0xFF);
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
bit_unpack_kernel(const uint8_t* __restrict__ in, T* __restrict__ out, long long n) {
    const long long byte = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long e0 = byte * 8;
    if (e0 >= n) return;
    const uint32_t bits = in[byte];
    if (e0 + 8 <= n && (reinterpret_cast<uintptr_t>(out + e0) % (8 * sizeof(T)) == 0)) {
        float f[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = (float)((bits >> j) & 1u);
        Pack<T, 8> p;
#pragma unroll
        for (int j = 0; j < 8; ++j) p.e[j] = from_f32<T>(f[j]);
        *reinterpret_cast<Pack<T, 8>*>(out + e0) = p;
    } else {
        for (int j = 0; j < 8 && e0 + j < n; ++j) out[e0 + j] = from_f32<T>((float)((bits >> j) & 1u));
    }
}

}  // namespace

at::Tensor bit_pack(const at::Tensor& x) {
    TORCH_CHECK(x.is_cuda(), "bit_pack: CUDA tensor required");
    const c10::cuda::CUDAGuard guard(x.device());
    at::Tensor xc = x.contiguous();
    const long long n = xc.numel();
    at::Tensor out = at::empty({(n + 7) / 8}, xc.options().dtype(at::kByte));
    if (n == 0) return out;
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    auto launch = [&](auto tag) {
        using T = decltype(tag);
        constexpr int V = 16 / sizeof(T);
        constexpr int ELEMS = V >= 8 ? V : 8;
        const long long threads = (n + ELEMS - 1) / ELEMS;
        bit_pack_kernel<T><<<(unsigned)((threads + kThreads - 1) / kThreads), kThreads, 0, st>>>(
            reinterpret_cast<const T*>(xc.data_ptr()), out.data_ptr<uint8_t>(), n);
    };
    switch (xc.scalar_type()) {
    case at::kFloat: launch(float{}); break;
    case at::kHalf: launch(__half{}); break;
    case at::kBFloat16: launch(__nv_bfloat16{}); break;
    default: TORCH_CHECK(false, "bit_pack: fp32 / fp16 / bf16 input required, got ", xc.scalar_type());
    }
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return out;
}

at::Tensor bit_unpack(const at::Tensor& packed, int64_t n, at::ScalarType dtype) {
    TORCH_CHECK(packed.is_cuda() && packed.scalar_type() == at::kByte && packed.is_contiguous(), "bit_unpack: contiguous uint8 CUDA tensor required");
    TORCH_CHECK(packed.numel() * 8 >= n, "bit_unpack: packed tensor too short");
    const c10::cuda::CUDAGuard guard(packed.device());
    at::Tensor out = at::empty({n}, packed.options().dtype(dtype));
    if (n == 0) return out;
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    const long long threads = (n + 7) / 8;
    const unsigned grid = (unsigned)((threads + kThreads - 1) / kThreads);
    switch (dtype) {
    case at::kFloat: bit_unpack_kernel<float><<<grid, kThreads, 0, st>>>(packed.data_ptr<uint8_t>(), out.data_ptr<float>(), n); break;
    case at::kHalf: bit_unpack_kernel<__half><<<grid, kThreads, 0, st>>>(packed.data_ptr<uint8_t>(), reinterpret_cast<__half*>(out.data_ptr()), n); break;
    case at::kBFloat16: bit_unpack_kernel<__nv_bfloat16><<<grid, kThreads, 0, st>>>(packed.data_ptr<uint8_t>(), reinterpret_cast<__nv_bfloat16*>(out.data_ptr()), n); break;
    default: TORCH_CHECK(false, "bit_unpack: fp32 / fp16 / bf16 output required");
    }
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return out;
}

}  // namespace sjb200

TORCH_LIBRARY_FRAGMENT(sjb200, m) {
    m.def("bit_pack(Tensor x) -> Tensor");
    m.def("bit_unpack(Tensor packed, int n, ScalarType dtype) -> Tensor");
}
TORCH_LIBRARY_IMPL(sjb200, CUDA, m) {
    m.impl("bit_pack", &sjb200::bit_pack);
    m.impl("bit_unpack", &sjb200::bit_unpack);
}
