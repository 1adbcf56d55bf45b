// Shared device helpers for the sm_100a kernels: 128-bit vector IO with dtype
// conversion, error-status words, bounded waits.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>

namespace sjb200 {

// ---- scalar conversion ------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_fp8_e4m3>(__nv_fp8_e4m3 v) { return float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_fp8_e5m2>(__nv_fp8_e5m2 v) { return float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __nv_fp8_e4m3 from_f32<__nv_fp8_e4m3>(float v) { return __nv_fp8_e4m3(v); }
template <> __device__ __forceinline__ __nv_fp8_e5m2 from_f32<__nv_fp8_e5m2>(float v) { return __nv_fp8_e5m2(v); }

// ---- V consecutive elements <-> float registers -----------------------------
// V * sizeof(T) is 16 bytes on the vector path and sizeof(T) on the scalar path.
template <typename T, int V> struct alignas(sizeof(T) * V) Pack { T e[V]; };

template <typename T, int V>
__device__ __forceinline__ void load_vec(const T* __restrict__ p, float (&out)[V]) {
    Pack<T, V> raw = *reinterpret_cast<const Pack<T, V>*>(p);
#pragma unroll
    for (int i = 0; i < V; ++i) out[i] = to_f32<T>(raw.e[i]);
}
// streaming variant: data read once, keep it out of L1
template <typename T, int V>
__device__ __forceinline__ void load_vec_stream(const T* __restrict__ p, float (&out)[V]) {
    Pack<T, V> raw;
    if constexpr (sizeof(T) * V == 16) {
        int4 r = __ldcs(reinterpret_cast<const int4*>(p));
        raw = *reinterpret_cast<Pack<T, V>*>(&r);
    } else if constexpr (sizeof(T) * V == 8) {
        int2 r = __ldcs(reinterpret_cast<const int2*>(p));
        raw = *reinterpret_cast<Pack<T, V>*>(&r);
    } else {
        raw = *reinterpret_cast<const Pack<T, V>*>(p);
    }
#pragma unroll
    for (int i = 0; i < V; ++i) out[i] = to_f32<T>(raw.e[i]);
}
template <typename T, int V>
__device__ __forceinline__ void store_vec(T* __restrict__ p, const float (&in)[V]) {
    Pack<T, V> raw;
#pragma unroll
    for (int i = 0; i < V; ++i) raw.e[i] = from_f32<T>(in[i]);
    if constexpr (sizeof(T) * V == 16) {
        __stcs(reinterpret_cast<int4*>(p), *reinterpret_cast<int4*>(&raw));
    } else if constexpr (sizeof(T) * V == 8) {
        __stcs(reinterpret_cast<int2*>(p), *reinterpret_cast<int2*>(&raw));
    } else {
        *reinterpret_cast<Pack<T, V>*>(p) = raw;
    }
}

// raw (unconverted) vector load: keeps V elements in V*sizeof(T)/4 registers until they are needed
template <typename T, int V>
__device__ __forceinline__ Pack<T, V> load_raw_stream(const T* __restrict__ p) {
    Pack<T, V> raw;
    if constexpr (sizeof(T) * V == 16) {
        int4 r = __ldcs(reinterpret_cast<const int4*>(p));
        raw = *reinterpret_cast<Pack<T, V>*>(&r);
    } else if constexpr (sizeof(T) * V == 8) {
        int2 r = __ldcs(reinterpret_cast<const int2*>(p));
        raw = *reinterpret_cast<Pack<T, V>*>(&r);
    } else {
        raw = *reinterpret_cast<const Pack<T, V>*>(p);
    }
    return raw;
}
template <typename T, int V>
__device__ __forceinline__ void unpack(const Pack<T, V>& raw, float (&out)[V]) {
#pragma unroll
    for (int i = 0; i < V; ++i) out[i] = to_f32<T>(raw.e[i]);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

}  // namespace sjb200
