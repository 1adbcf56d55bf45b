// BatchNorm batch statistics without any allocation: the per-block partial sums live in a
// file-scope device array, and the last block to finish adds them up (in a fixed order, in
// double precision) and writes the coefficients.  See bn_stats_noalloc.h for the contract.
#include "bn_stats_noalloc.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kMaxC = SJB200_BN_NOALLOC_MAX_CHANNELS;
constexpr int kMaxBlocks = SJB200_BN_NOALLOC_MAX_BLOCKS;
constexpr int kMaxDevices = 64;

// Layout: [kMaxBlocks][2][channels] partial sums, then (at float index kCounterAt) the arrival counter.
constexpr size_t kCounterAt = (size_t)kMaxBlocks * 2 * kMaxC;
static __device__ __align__(256) float g_bn_noalloc_scratch[kCounterAt + 64];

template <typename T>
__global__ void __launch_bounds__(kThreads)
bn_stats_noalloc_kernel(const T* __restrict__ y, long long rows, int C, const float* __restrict__ gamma,
                        const float* __restrict__ beta, float eps, float* __restrict__ mean_out,
                        float* __restrict__ invstd_out, float* __restrict__ scale, float* __restrict__ shift,
                        float* __restrict__ scratch) {
    __shared__ float s_buf[2 * kThreads * 8];          // [rows in flight][2][channels of this block's pass]
    __shared__ unsigned s_ticket;
    const int G = C / 8;                               // 8-channel groups; G <= 256 because C <= 2048
    const int tpr = G < kThreads ? G : kThreads;       // threads per row
    const int rpi = kThreads / tpr;                    // rows in flight
    const int rl = threadIdx.x / tpr, cl = threadIdx.x % tpr;
    const long long per_block = (rows + gridDim.x - 1) / gridDim.x;
    const long long r0 = per_block * blockIdx.x;
    const long long r1 = r0 + per_block < rows ? r0 + per_block : rows;

    float s1[8], s2[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { s1[j] = 0.0f; s2[j] = 0.0f; }
    if (rl < rpi) {
        for (long long r = r0 + rl; r < r1; r += rpi) {
            float v[8];
            sjb200::load_vec_stream<T, 8>(y + r * C + cl * 8, v);
#pragma unroll
            for (int j = 0; j < 8; ++j) { s1[j] += v[j]; s2[j] += v[j] * v[j]; }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            s_buf[(rl * 2 + 0) * C + cl * 8 + j] = s1[j];
            s_buf[(rl * 2 + 1) * C + cl * 8 + j] = s2[j];
        }
    }
    __syncthreads();
    float* mine = scratch + (size_t)blockIdx.x * 2 * C;
    for (int i = threadIdx.x; i < 2 * C; i += kThreads) {
        const int which = i / C, c = i % C;
        float acc = 0.0f;
        for (int r = 0; r < rpi; ++r) acc += s_buf[(r * 2 + which) * C + c];
        mine[i] = acc;
    }
    // publish this block's partials, then take a ticket; the holder of the last ticket finalises
    __threadfence();
    __syncthreads();
    unsigned* counter = reinterpret_cast<unsigned*>(scratch + kCounterAt);
    if (threadIdx.x == 0) s_ticket = atomicAdd(counter, 1u);
    __syncthreads();
    if (s_ticket != gridDim.x - 1) return;
    __threadfence();
    const double count = (double)rows;
    for (int c = threadIdx.x; c < C; c += kThreads) {
        double a1 = 0.0, a2 = 0.0;
        for (unsigned b = 0; b < gridDim.x; ++b) {
            a1 += (double)__ldcg(scratch + (size_t)b * 2 * C + c);
            a2 += (double)__ldcg(scratch + (size_t)b * 2 * C + C + c);
        }
        const double mean = a1 / count;
        double var = a2 / count - mean * mean;
        if (var < 0.0) var = 0.0;
        const float invstd = (float)(1.0 / sqrt(var + (double)eps));
        const float g = gamma != nullptr ? gamma[c] : 1.0f, b0 = beta != nullptr ? beta[c] : 0.0f;
        mean_out[c] = (float)mean;
        invstd_out[c] = invstd;
        scale[c] = g * invstd;
        shift[c] = b0 - (float)mean * g * invstd;
    }
}

thread_local char t_error[256] = "";

int fail(int code, const char* what, cudaError_t err = cudaSuccess) {
    if (err != cudaSuccess) std::snprintf(t_error, sizeof(t_error), "%s: %s", what, cudaGetErrorString(err));
    else std::snprintf(t_error, sizeof(t_error), "%s", what);
    return code;
}

// Device address of the scratch array, resolved once per device with that device current.
std::mutex g_setup_mutex;
float* g_scratch_ptr[kMaxDevices] = {};

int scratch_for_current_device(float** out, int* device_out) {
    int dev = -1;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return fail(SJB200_NOALLOC_E_SETUP, "cudaGetDevice", err);
    if (dev < 0 || dev >= kMaxDevices) return fail(SJB200_NOALLOC_E_SETUP, "device ordinal out of range");
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_ptr[dev] == nullptr) {
        float* ptr = nullptr;
        err = cudaGetSymbolAddress((void**)&ptr, g_bn_noalloc_scratch);
        if (err != cudaSuccess || ptr == nullptr) return fail(SJB200_NOALLOC_E_SETUP, "cudaGetSymbolAddress(scratch)", err);
        g_scratch_ptr[dev] = ptr;
    }
    *out = g_scratch_ptr[dev];
    *device_out = dev;
    return SJB200_NOALLOC_OK;
}

}  // namespace

extern "C" SJB200_EXPORT int sjb200_bn_stats_noalloc(const void* y, int dtype, long long rows, int channels, const float* gamma,
                                       const float* beta, float eps, float* mean, float* invstd, float* scale, float* shift,
                                       void* stream) {
    t_error[0] = '\0';
    if (y == nullptr || mean == nullptr || invstd == nullptr || scale == nullptr || shift == nullptr)
        return fail(SJB200_NOALLOC_E_BAD_ARGUMENT, "null input or output pointer");
    if (rows <= 0 || channels <= 0 || channels % 8 != 0)
        return fail(SJB200_NOALLOC_E_BAD_ARGUMENT, "rows must be positive and channels a positive multiple of 8");
    if (dtype < 0 || dtype > 2) return fail(SJB200_NOALLOC_E_BAD_ARGUMENT, "dtype must be 0 (fp32), 1 (fp16) or 2 (bf16)");
    if (channels > kMaxC) {
        std::snprintf(t_error, sizeof(t_error), "channels = %d exceeds the fixed scratch capacity of %d channels", channels, kMaxC);
        return SJB200_NOALLOC_E_TOO_LARGE;
    }
    const size_t vec_bytes = 8 * (dtype == 0 ? sizeof(float) : sizeof(__half));   // one 8-channel vector load
    if (reinterpret_cast<uintptr_t>(y) % vec_bytes != 0)
        return fail(SJB200_NOALLOC_E_BAD_ARGUMENT, "y must be aligned to 8 elements (32 bytes for fp32, 16 for fp16/bf16)");

    float* scratch = nullptr;
    int dev = -1;
    const int rc = scratch_for_current_device(&scratch, &dev);
    if (rc != SJB200_NOALLOC_OK) return rc;

    // Every operand must be memory the kernel may dereference: device memory of the current device, or managed
    // memory.  Host and unregistered pointers are refused here, before anything is launched.
    const struct { const void* ptr; const char* name; } operands[] = {
        {y, "y"}, {mean, "mean"}, {invstd, "invstd"}, {scale, "scale"}, {shift, "shift"}, {gamma, "gamma"}, {beta, "beta"}};
    cudaError_t err = cudaSuccess;
    for (const auto& op : operands) {
        if (op.ptr == nullptr) continue;                      // gamma / beta are optional
        cudaPointerAttributes attr{};
        err = cudaPointerGetAttributes(&attr, op.ptr);
        if (err != cudaSuccess) {
            std::snprintf(t_error, sizeof(t_error), "cudaPointerGetAttributes(%s): %s", op.name, cudaGetErrorString(err));
            return SJB200_NOALLOC_E_BAD_ARGUMENT;
        }
        if (attr.type == cudaMemoryTypeManaged) continue;
        if (attr.type != cudaMemoryTypeDevice) {
            std::snprintf(t_error, sizeof(t_error), "%s is not device memory (host or unregistered pointer)", op.name);
            return SJB200_NOALLOC_E_BAD_ARGUMENT;
        }
        if (attr.device != dev) {
            std::snprintf(t_error, sizeof(t_error), "%s lives on device %d, the current device is %d", op.name, attr.device, dev);
            return SJB200_NOALLOC_E_WRONG_DEVICE;
        }
    }

    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    // the arrival counter is the only part of the scratch that must start at zero
    err = cudaMemsetAsync(scratch + kCounterAt, 0, sizeof(unsigned), st);
    if (err != cudaSuccess) return fail(SJB200_NOALLOC_E_LAUNCH, "cudaMemsetAsync(counter)", err);

    long long want = (rows + 63) / 64;                 // at least 64 rows per block
    const int grid = (int)(want < 1 ? 1 : (want > kMaxBlocks ? kMaxBlocks : want));
    switch (dtype) {
    case 0:
        bn_stats_noalloc_kernel<float><<<grid, kThreads, 0, st>>>(static_cast<const float*>(y), rows, channels, gamma, beta, eps,
                                                                  mean, invstd, scale, shift, scratch);
        break;
    case 1:
        bn_stats_noalloc_kernel<__half><<<grid, kThreads, 0, st>>>(static_cast<const __half*>(y), rows, channels, gamma, beta, eps,
                                                                   mean, invstd, scale, shift, scratch);
        break;
    default:
        bn_stats_noalloc_kernel<__nv_bfloat16><<<grid, kThreads, 0, st>>>(static_cast<const __nv_bfloat16*>(y), rows, channels, gamma,
                                                                          beta, eps, mean, invstd, scale, shift, scratch);
        break;
    }
    err = cudaGetLastError();
    if (err != cudaSuccess) return fail(SJB200_NOALLOC_E_LAUNCH, "kernel launch", err);
    return SJB200_NOALLOC_OK;
}

extern "C" SJB200_EXPORT const char* sjb200_noalloc_last_error(void) { return t_error; }
