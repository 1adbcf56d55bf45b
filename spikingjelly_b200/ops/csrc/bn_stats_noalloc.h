// C entry point for BatchNorm batch statistics that performs no memory allocation of any kind.
//
// This entry point has no counterpart in the SpikingJelly reference; it exists for hosts that
// cannot, or must not, allocate device memory at call time:
//   * programs that are not PyTorch programs (plain C/C++ hosts, or Python through ctypes) and
//     therefore have no caching allocator to take a scratch buffer from;
//   * servers that hand the whole device to an arena of their own at start-up, where a later
//     cudaMalloc can fail although the arena has room;
//   * latency-critical loops, because cudaMalloc and cudaFree may synchronise the whole device
//     and stall unrelated streams.
// The regular PyTorch operator `sjb200::bn_coefficients` takes its per-block partial-sum buffer
// from torch's allocator on every call; this variant keeps that buffer in a fixed array inside
// the library image instead.
//
// Contract
//   * The scratch array is ONE per device and is shared by every call on that device, from any
//     stream or thread.  Two calls whose execution may overlap on the same device race on it and
//     produce wrong statistics: serialise them (same stream, or an event between streams).
//   * The first call on each device performs one-time set-up (it looks up the device address of
//     the scratch array).  Make that first call during initialisation, before any stream capture
//     is begun on the calling thread.
//   * Limits: channels must be a multiple of 8 and at most SJB200_BN_NOALLOC_MAX_CHANNELS; any
//     number of rows.  Larger channel counts are rejected with SJB200_NOALLOC_E_TOO_LARGE; nothing
//     is launched in that case.
//   * `y` is a dense channels-last matrix [rows, channels] on the CURRENT device; gamma/beta may
//     be null (treated as 1 and 0); mean/invstd/scale/shift are fp32 [channels] outputs with
//       mean = E[y], invstd = 1/sqrt(Var[y] + eps) (biased variance),
//       scale = gamma * invstd, shift = beta - mean * scale.
//   * The work is enqueued on `stream` (a cudaStream_t passed as void*; null = default stream)
//     and the function returns without waiting for it.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// exported from the shared library although the library is built with hidden visibility
#define SJB200_EXPORT __attribute__((visibility("default")))

#define SJB200_BN_NOALLOC_MAX_CHANNELS 2048
#define SJB200_BN_NOALLOC_MAX_BLOCKS 148
// scratch held in the library image: MAX_BLOCKS * 2 * MAX_CHANNELS floats (about 2.3 MiB) + one counter

enum {
    SJB200_NOALLOC_OK = 0,
    SJB200_NOALLOC_E_BAD_ARGUMENT = -1,   // null / host / unregistered pointer, rows <= 0, channels not a multiple of 8, unknown dtype
    SJB200_NOALLOC_E_TOO_LARGE = -2,      // channels > SJB200_BN_NOALLOC_MAX_CHANNELS
    SJB200_NOALLOC_E_SETUP = -3,          // the scratch symbol could not be resolved on this device
    SJB200_NOALLOC_E_LAUNCH = -4,         // the CUDA runtime refused the memset or the launch
    SJB200_NOALLOC_E_WRONG_DEVICE = -5    // an operand lives on a device other than the current one
};

// dtype: 0 = float32, 1 = float16, 2 = bfloat16
SJB200_EXPORT int sjb200_bn_stats_noalloc(const void* y, int dtype, long long rows, int channels, const float* gamma, const float* beta,
                            float eps, float* mean, float* invstd, float* scale, float* shift, void* stream);

// Text of the most recent failure on the calling thread ("" if none).
SJB200_EXPORT const char* sjb200_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
