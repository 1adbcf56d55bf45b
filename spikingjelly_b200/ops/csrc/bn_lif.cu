// BatchNorm (training statistics or frozen) fused with the multi-step neuron, for
// channels-last activations [T, R, C] (C contiguous).
//
//   forward :  stats(y) -> (scale, shift) ;  spikes = LIF_T(y * scale[c] + shift[c]) (+ residual)
//   backward:  pass 1  recomputes the membrane trajectory, runs BPTT and writes g = dL/d(BN out)
//                      while accumulating sum(g) and sum(g * xhat) per channel;
//              pass 2  dy = A[c] g + B[c] y + D[c]   (the BN backward in closed form)
// The normalised tensor never exists in memory.  Per-channel reductions use per-block partial
// sums in a scratch buffer that a finalize kernel adds in a fixed order (deterministic).
#include <ATen/ATen.h>
#include <cstdlib>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "bn_lif.h"
#include "neuron_scan.cuh"

namespace sjb200 {
namespace {

constexpr int kThreads = 256;
constexpr int TCB = 4;   // steps per register-resident chunk in the fused kernels

// ----------------------------------------------------------------- statistics
// partial[blk][0][c] = sum of y over the block's rows, partial[blk][1][c] = sum of squares.
// Threads that share a channel group write their private sums to shared memory and one thread
// per channel adds them in a fixed order, so the result does not depend on scheduling.
template <typename T>
__global__ void __launch_bounds__(kThreads)
bn_stats_partial_kernel(const T* __restrict__ y, long long rows, int C, float* __restrict__ partial) {
    extern __shared__ float s_buf[];   // [rpi][2][Cs] with Cs = min(C, 8 * blockDim)
    const int G = C / 8;
    const int tpr = G < (int)blockDim.x ? G : (int)blockDim.x;
    const int rpi = blockDim.x / tpr;
    const int rl = threadIdx.x / tpr, cl = threadIdx.x % tpr;
    const int Cs = tpr * 8;
    const long long rows_per_block = (rows + gridDim.x - 1) / gridDim.x;
    const long long r0 = rows_per_block * blockIdx.x;
    const long long r1 = r0 + rows_per_block < rows ? r0 + rows_per_block : rows;
    float* out = partial + (size_t)blockIdx.x * 2 * C;
    for (int cg0 = 0; cg0 < G; cg0 += tpr) {          // one pass unless C > 8 * blockDim
        const int cg = cg0 + cl;
        float s1[8], s2[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) { s1[j] = 0.0f; s2[j] = 0.0f; }
        if (rl < rpi && cg < G) {
            for (long long r = r0 + rl; r < r1; r += rpi) {
                float v[8];
                load_vec_stream<T, 8>(y + r * C + cg * 8, v);
#pragma unroll
                for (int j = 0; j < 8; ++j) { s1[j] += v[j]; s2[j] += v[j] * v[j]; }
            }
        }
        if (rl < rpi) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                s_buf[(rl * 2 + 0) * Cs + cl * 8 + j] = s1[j];
                s_buf[(rl * 2 + 1) * Cs + cl * 8 + j] = s2[j];
            }
        }
        __syncthreads();
        for (int i = threadIdx.x; i < 2 * Cs; i += blockDim.x) {
            const int which = i / Cs, cc = i % Cs;
            if (cg0 * 8 + cc < C) {
                float acc = 0.0f;
                for (int r = 0; r < rpi; ++r) acc += s_buf[(r * 2 + which) * Cs + cc];
                out[which * C + cg0 * 8 + cc] = acc;
            }
        }
        __syncthreads();
    }
}

// Sum partial[b][which][c] over b for 8 channels per block: 32 slices of blocks are summed by
// different threads and combined in a fixed order (deterministic), instead of one long serial loop.
constexpr int kFinCh = 8, kFinSlices = 32;     // blockDim.x == kFinCh * kFinSlices == 256
__device__ __forceinline__ void reduce_partials(const float* __restrict__ partial, int nblk, int C, int c,
                                                double& s1, double& s2) {
    __shared__ double sh1[kFinSlices][kFinCh], sh2[kFinSlices][kFinCh];
    const int lane_c = threadIdx.x % kFinCh, slice = threadIdx.x / kFinCh;
    double a1 = 0.0, a2 = 0.0;
    if (c < C) {
        // sixteen independent loads per round: the serial chain is nblk / 256 memory latencies, not nblk / 32
        int b = slice;
        for (; b + 7 * kFinSlices < nblk; b += 8 * kFinSlices) {
            float p1[8], p2[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                p1[u] = partial[(size_t)(b + u * kFinSlices) * 2 * C + c];
                p2[u] = partial[(size_t)(b + u * kFinSlices) * 2 * C + C + c];
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) { a1 += (double)p1[u]; a2 += (double)p2[u]; }
        }
        for (; b < nblk; b += kFinSlices) {
            a1 += (double)partial[(size_t)b * 2 * C + c];
            a2 += (double)partial[(size_t)b * 2 * C + C + c];
        }
    }
    sh1[slice][lane_c] = a1;
    sh2[slice][lane_c] = a2;
    __syncthreads();
    s1 = 0.0; s2 = 0.0;
#pragma unroll 8
    for (int k = 0; k < kFinSlices; ++k) { s1 += sh1[k][lane_c]; s2 += sh2[k][lane_c]; }
}

// 8 channels per block: fixed-order sum of the block partials, then the BN coefficients
__global__ void bn_finalize_forward_kernel(const float* __restrict__ partial, int nblk, int C, double count, float eps,
                                           float momentum, const float* __restrict__ gamma, const float* __restrict__ beta,
                                           float* __restrict__ running_mean, float* __restrict__ running_var,
                                           float* __restrict__ mean_out, float* __restrict__ invstd_out,
                                           float* __restrict__ scale, float* __restrict__ shift) {
    const int c = blockIdx.x * kFinCh + threadIdx.x % kFinCh;
    double s1, s2;
    reduce_partials(partial, nblk, C, c, s1, s2);
    if (c >= C || threadIdx.x >= kFinCh) return;
    const double mean = s1 / count;
    double var = s2 / count - mean * mean;
    if (var < 0.0) var = 0.0;
    const float invstd = (float)(1.0 / sqrt(var + (double)eps));
    const float g = gamma != nullptr ? gamma[c] : 1.0f, b0 = beta != nullptr ? beta[c] : 0.0f;
    mean_out[c] = (float)mean;
    invstd_out[c] = invstd;
    scale[c] = g * invstd;
    shift[c] = b0 - (float)mean * g * invstd;
    if (running_mean != nullptr) {
        const double unbiased = count > 1.0 ? var * count / (count - 1.0) : var;
        running_mean[c] = (1.0f - momentum) * running_mean[c] + momentum * (float)mean;
        running_var[c] = (1.0f - momentum) * running_var[c] + momentum * (float)unbiased;
    }
}

// frozen statistics: scale/shift from the running estimates
__global__ void bn_frozen_coeff_kernel(int C, float eps, const float* __restrict__ gamma, const float* __restrict__ beta,
                                       const float* __restrict__ running_mean, const float* __restrict__ running_var,
                                       float* __restrict__ mean_out, float* __restrict__ invstd_out,
                                       float* __restrict__ scale, float* __restrict__ shift) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const float invstd = rsqrtf(running_var[c] + eps);
    const float g = gamma != nullptr ? gamma[c] : 1.0f, b0 = beta != nullptr ? beta[c] : 0.0f;
    mean_out[c] = running_mean[c];
    invstd_out[c] = invstd;
    scale[c] = g * invstd;
    shift[c] = b0 - running_mean[c] * g * invstd;
}

// -------------------------------------------------------------------- forward
// y, out, res: [T, N] with N = R * C; scale/shift: [C]; ckpt: [ceil(T/4) - 1, N] fp32 or null
// TFIX > 0: sequence length known at compile time and <= TCB (one register chunk, no checkpoints, no
// per-step bounds predicates); HAS_RES: a residual is added to the spikes.
template <typename T, int V, int KIND, int TFIX, bool HAS_RES>
__global__ void __launch_bounds__(kThreads, 3)
bn_lif_forward_kernel(ScanParams p_in, int C, const T* __restrict__ y, const float* __restrict__ scale,
                      const float* __restrict__ shift, const T* __restrict__ res, T* __restrict__ out,
                      float* __restrict__ ckpt) {
    ScanParams p = p_in;
    if constexpr (TFIX > 0) { p.T = TFIX; ckpt = nullptr; }
    const long long n0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * V;
    if (n0 >= p.N) return;
    const Neuron<KIND> nrn(p);
    const int c0 = (int)(n0 % C);
    float sc[V], sh[V], v[V];
    load_vec<float, V>(scale + c0, sc);
    load_vec<float, V>(shift + c0, sh);
#pragma unroll
    for (int j = 0; j < V; ++j) v[j] = p.v_init_scalar;
    for (int t0 = 0; t0 < p.T; t0 += TCB) {
        Pack<T, V> yr[TCB], rr[TCB];
#pragma unroll
        for (int i = 0; i < TCB; ++i) {
            if (t0 + i < p.T) {
                yr[i] = load_raw_stream<T, V>(y + (long long)(t0 + i) * p.N + n0);
                if constexpr (HAS_RES) rr[i] = load_raw_stream<T, V>(res + (long long)(t0 + i) * p.N + n0);
            }
        }
#pragma unroll
        for (int i = 0; i < TCB; ++i) {
            if (t0 + i < p.T) {
                float x[V], s[V];
                unpack<T, V>(yr[i], x);
#pragma unroll
                for (int j = 0; j < V; ++j) {
                    const float h = nrn.charge(fmaf(x[j], sc[j], sh[j]), v[j]);
                    const bool f = nrn.fire(h);
                    v[j] = nrn.reset(h, f);
                    s[j] = f ? 1.0f : 0.0f;
                }
                if constexpr (HAS_RES) {
                    float r[V];
                    unpack<T, V>(rr[i], r);
#pragma unroll
                    for (int j = 0; j < V; ++j) s[j] += r[j];
                }
                store_vec<T, V>(out + (long long)(t0 + i) * p.N + n0, s);
            }
        }
        if (ckpt != nullptr && t0 + TCB < p.T) store_vec<float, V>(ckpt + (long long)(t0 / TCB) * p.N + n0, v);
    }
}

// ------------------------------------------------------------ backward, pass 1
// g_out: dL/d(out) [T, N];  writes gx = dL/d(BN output) [T, N];
// partial[blk][0][c] = sum gx, partial[blk][1][c] = sum gx * y   (the finalize kernel turns the latter
// into sum gx * xhat = invstd * (sum gx y - mean * sum gx))
template <typename T, int V, int KIND, int TFIX = 0, int OCC = 2>
__global__ void __launch_bounds__(kThreads, OCC)
bn_lif_backward1_kernel(ScanParams p_in, int C, const T* __restrict__ y, const T* __restrict__ g_out,
                        const float* __restrict__ scale, const float* __restrict__ shift,
                        const float* __restrict__ ckpt, T* __restrict__ gx_out, float* __restrict__ partial) {
    // The host picks gridDim so that (gridDim * blockDim * V) % C == 0: a thread then sees the same
    // channels in every iteration of its grid-stride loop and keeps its sums in registers.
    extern __shared__ float s_buf[];   // [blockDim][2 V]
    // TFIX > 0: the sequence length is a compile-time constant that fits one register chunk
    // (no checkpoints, no per-step bounds predicates)
    ScanParams p = p_in;
    if constexpr (TFIX > 0) p.T = TFIX;
    const Neuron<KIND> nrn(p);
    const float dhdx = nrn.dh_dx();
    const float dhdv = nrn.dh_dv(0.0f);
    const float kd = p.detach_reset ? 0.0f : 1.0f;
    const float k_s = p.soft_reset ? 0.0f : 1.0f;
    const float k_a = kd * (p.soft_reset ? -p.v_th : p.v_reset);
    const float k_b = kd * (p.soft_reset ? 0.0f : -1.0f);
    const long long n_vec = p.N / V;
    const int n_chunks = (p.T + TCB - 1) / TCB;
    const long long first = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int c0 = (int)((first * V) % C);
    float sc[V], sh[V], a1[V], a2[V];
    load_vec<float, V>(scale + c0, sc);
    load_vec<float, V>(shift + c0, sh);
#pragma unroll
    for (int j = 0; j < V; ++j) { a1[j] = 0.0f; a2[j] = 0.0f; }
    for (long long vec = first; vec < n_vec; vec += (long long)gridDim.x * blockDim.x) {
        const long long n0 = vec * V;
        float c[V];
#pragma unroll
        for (int j = 0; j < V; ++j) c[j] = 0.0f;
        for (int ck = n_chunks - 1; ck >= 0; --ck) {
            const int t0 = ck * TCB;
            float v0[V];
            if (ck > 0) load_vec<float, V>(ckpt + (long long)(ck - 1) * p.N + n0, v0);
            else {
#pragma unroll
                for (int j = 0; j < V; ++j) v0[j] = p.v_init_scalar;
            }
            Pack<T, V> yr[TCB], gr[TCB];
#pragma unroll
            for (int i = 0; i < TCB; ++i) {
                if (t0 + i < p.T) {
                    yr[i] = load_raw_stream<T, V>(y + (long long)(t0 + i) * p.N + n0);
                    gr[i] = load_raw_stream<T, V>(g_out + (long long)(t0 + i) * p.N + n0);
                }
            }
            float h[TCB][V];
            {
                float v[V];
#pragma unroll
                for (int j = 0; j < V; ++j) v[j] = v0[j];
#pragma unroll
                for (int i = 0; i < TCB; ++i) {
                    if (t0 + i < p.T) {
                        float yv[V];
                        unpack<T, V>(yr[i], yv);
#pragma unroll
                        for (int j = 0; j < V; ++j) {
                            const float hh = nrn.charge(fmaf(yv[j], sc[j], sh[j]), v[j]);
                            h[i][j] = hh;
                            v[j] = nrn.reset(hh, nrn.fire(hh));
                        }
                    }
                }
            }
#pragma unroll
            for (int i = TCB - 1; i >= 0; --i) {
                if (t0 + i < p.T) {
                    const long long off = (long long)(t0 + i) * p.N + n0;
                    float gs[V], sg[V], gx[V], yv[V];
                    unpack<T, V>(gr[i], gs);
                    unpack<T, V>(yr[i], yv);
#pragma unroll
                    for (int j = 0; j < V; ++j) sg[j] = h[i][j] - p.v_th;
                    surrogate_grad_vec<V>(p.sg_id, sg, p.sg_p0, p.sg_p1);
#pragma unroll
                    for (int j = 0; j < V; ++j) {
                        const float hh = h[i][j];
                        const float s = nrn.fire(hh) ? 1.0f : 0.0f;
                        const float dv_dh = fmaf(sg[j], fmaf(k_b, hh, k_a), fmaf(-k_s, s, 1.0f));
                        const float gh = fmaf(gs[j], sg[j], c[j] * dv_dh);
                        c[j] = gh * dhdv;
                        gx[j] = gh * dhdx;
                        a1[j] += gx[j];
                        a2[j] = fmaf(gx[j], yv[j], a2[j]);
                    }
                    store_vec<T, V>(gx_out + off, gx);
                }
            }
        }
    }
    // deterministic block reduction: thread t owns channel group (g0 + t) mod G
#pragma unroll
    for (int j = 0; j < V; ++j) {
        s_buf[threadIdx.x * 2 * V + j] = a1[j];
        s_buf[threadIdx.x * 2 * V + V + j] = a2[j];
    }
    __syncthreads();
    const int G = C / V;
    const int g0 = (int)(((long long)blockIdx.x * blockDim.x) % G);
    float* outp = partial + (size_t)blockIdx.x * 2 * C;
    for (int i = threadIdx.x; i < 2 * C; i += blockDim.x) {
        const int which = i / C, ch = i % C;
        const int grp = ch / V, j = ch % V;
        const int f = ((grp - g0) % G + G) % G;     // first thread of the block that owns this group
        float acc = 0.0f;
        for (int t = f; t < (int)blockDim.x; t += G) acc += s_buf[t * 2 * V + which * V + j];
        outp[i] = acc;
    }
}

// per channel: grad_gamma, grad_beta and the coefficients of pass 2
__global__ void bn_finalize_backward_kernel(const float* __restrict__ partial, int nblk, int C, double count, int training,
                                            const float* __restrict__ gamma, const float* __restrict__ mean,
                                            const float* __restrict__ invstd, float* __restrict__ grad_gamma,
                                            float* __restrict__ grad_beta, float* __restrict__ coefA,
                                            float* __restrict__ coefB, float* __restrict__ coefD) {
    const int c = blockIdx.x * kFinCh + threadIdx.x % kFinCh;
    double s1, s2;
    reduce_partials(partial, nblk, C, c, s1, s2);
    if (c >= C || threadIdx.x >= kFinCh) return;
    s2 = (double)invstd[c] * (s2 - (double)mean[c] * s1);   // sum gx * xhat
    grad_beta[c] = (float)s1;
    grad_gamma[c] = (float)s2;
    const float g = gamma != nullptr ? gamma[c] : 1.0f;
    const float A = g * invstd[c];
    if (training) {
        const float mg = (float)(s1 / count), mgx = (float)(s2 / count);
        coefA[c] = A;
        coefB[c] = -A * mgx * invstd[c];
        coefD[c] = -A * mg + A * mgx * invstd[c] * mean[c];
    } else {   // frozen statistics: BN is a fixed affine map
        coefA[c] = A; coefB[c] = 0.0f; coefD[c] = 0.0f;
    }
}

// ------------------------------------------------------------ backward, pass 2
template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
bn_backward2_kernel(long long total, int C, const T* __restrict__ gx, const T* __restrict__ y,
                    const float* __restrict__ coefA, const float* __restrict__ coefB, const float* __restrict__ coefD,
                    T* __restrict__ dy) {
    const long long n0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * V;
    if (n0 >= total) return;
    const int c0 = (int)(n0 % C);
    float a[V], b[V], d[V], g[V], yy[V], o[V];
    load_vec<float, V>(coefA + c0, a);
    load_vec<float, V>(coefB + c0, b);
    load_vec<float, V>(coefD + c0, d);
    load_vec_stream<T, V>(gx + n0, g);
    load_vec_stream<T, V>(y + n0, yy);
#pragma unroll
    for (int j = 0; j < V; ++j) o[j] = fmaf(a[j], g[j], fmaf(b[j], yy[j], d[j]));
    store_vec<T, V>(dy + n0, o);
}

#define SJ_BN_DISPATCH(DTYPE, ...)                                                         \
    switch (DTYPE) {                                                                        \
    case at::kFloat: { using scalar_t = float; __VA_ARGS__; break; }                        \
    case at::kHalf: { using scalar_t = __half; __VA_ARGS__; break; }                        \
    case at::kBFloat16: { using scalar_t = __nv_bfloat16; __VA_ARGS__; break; }             \
    default: TORCH_CHECK(false, "bn_lif: unsupported dtype ", DTYPE);                       \
    }
#define SJ_BN_KIND(KIND_VALUE, ...)                                                          \
    switch (KIND_VALUE) {                                                                    \
    case NK_IF: { constexpr int KIND = NK_IF; __VA_ARGS__; break; }                          \
    case NK_LIF_DI: { constexpr int KIND = NK_LIF_DI; __VA_ARGS__; break; }                  \
    case NK_LIF_NDI: { constexpr int KIND = NK_LIF_NDI; __VA_ARGS__; break; }                \
    default: TORCH_CHECK(false, "bn_lif: neuron kind ", KIND_VALUE, " has no fused form");   \
    }

int stats_grid(long long rows) {
    const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    const long long want = (rows + 31) / 32;
    return (int)std::max<long long>(1, std::min<long long>(want, (long long)sms * 2));
}

ScanParams lif_params(int64_t T, int64_t N, int64_t kind, double tau, double v_th, double v_reset, bool soft,
                      double v_init) {
    ScanParams p{};
    p.T = (int)T; p.N = N; p.kind = (int)kind; p.inv_tau = 1.0f / (float)tau;
    p.v_th = (float)v_th; p.v_reset = (float)v_reset; p.soft_reset = soft ? 1 : 0;
    p.v_init = nullptr; p.v_init_scalar = (float)v_init; p.r_ptr = nullptr;
    return p;
}

}  // namespace

void launch_bn_finalize_backward(const float* partial, int nblk, int C, double count, int training, const float* gamma,
                                 const float* mean, const float* invstd, float* grad_gamma, float* grad_beta, float* coefA,
                                 float* coefB, float* coefD, cudaStream_t stream) {
    bn_finalize_backward_kernel<<<(C + kFinCh - 1) / kFinCh, kFinCh * kFinSlices, 0, stream>>>(partial, nblk, C, count, training, gamma, mean, invstd,
                                                                  grad_gamma, grad_beta, coefA, coefB, coefD);
}

// Training-mode or frozen BN coefficients of a channels-last tensor y [*, C].
// returns (mean, invstd, scale, shift) fp32 [C]; updates running stats in place when training.
// partial [nblk, 2, C] -> out [gridDim.x, 2, C]: block b sums rows [b * per, (b + 1) * per) in order (deterministic).  Used
// when a producer emits so many partial rows that the per-channel finalisation (C / 8 blocks) would be the slow part.
__global__ void __launch_bounds__(256)
bn_partial_fold_kernel(const float* __restrict__ partial, int nblk, int width, int per, float* __restrict__ out) {
    const int r0 = blockIdx.x * per, r1 = min(nblk, r0 + per);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
        int r = r0;
        for (; r + 3 < r1; r += 4) {
            a0 += partial[(size_t)r * width + i];
            a1 += partial[(size_t)(r + 1) * width + i];
            a2 += partial[(size_t)(r + 2) * width + i];
            a3 += partial[(size_t)(r + 3) * width + i];
        }
        for (; r < r1; ++r) a0 += partial[(size_t)r * width + i];
        out[(size_t)blockIdx.x * width + i] = (a0 + a1) + (a2 + a3);
    }
}

// mean / invstd / scale / shift from partial sums [nblk, 2, C] that some other kernel produced (the tensor-core GEMM's
// epilogue emits this layout); `rows` is the number of values per channel behind them.
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> bn_coefficients_partial(
    const at::Tensor& partial, int64_t rows, const c10::optional<at::Tensor>& gamma, const c10::optional<at::Tensor>& beta,
    const c10::optional<at::Tensor>& running_mean, const c10::optional<at::Tensor>& running_var, double momentum, double eps) {
    TORCH_CHECK(partial.is_cuda() && partial.is_contiguous() && partial.dim() == 3 && partial.size(1) == 2 &&
                partial.scalar_type() == at::kFloat, "bn_coefficients_partial: contiguous fp32 CUDA [blocks, 2, C] required");
    const c10::cuda::CUDAGuard guard(partial.device());
    const int C = (int)partial.size(2);
    int nblk = (int)partial.size(0);
    auto fopt = partial.options();
    cudaStream_t stream0 = at::cuda::getCurrentCUDAStream();
    at::Tensor folded;
    const float* pptr = partial.data_ptr<float>();
    if (nblk > 2048) {
        const int rows_out = 512, per = (nblk + rows_out - 1) / rows_out;
        const int used = (nblk + per - 1) / per;
        folded = at::empty({used, 2, C}, fopt);
        bn_partial_fold_kernel<<<used, 256, 0, stream0>>>(pptr, nblk, 2 * C, per, folded.data_ptr<float>());
        C10_CUDA_KERNEL_LAUNCH_CHECK();
        pptr = folded.data_ptr<float>();
        nblk = used;
    }
    at::Tensor mean = at::empty({C}, fopt), invstd = at::empty({C}, fopt), scale = at::empty({C}, fopt), shift = at::empty({C}, fopt);
    auto fptr = [](const c10::optional<at::Tensor>& t) -> float* {
        if (!t.has_value() || !t->defined()) return nullptr;
        TORCH_CHECK(t->scalar_type() == at::kFloat && t->is_contiguous(), "BN parameters and buffers must be contiguous fp32");
        return t->data_ptr<float>();
    };
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    bn_finalize_forward_kernel<<<(C + kFinCh - 1) / kFinCh, kFinCh * kFinSlices, 0, stream>>>(
        pptr, nblk, C, (double)rows, (float)eps, (float)momentum, fptr(gamma), fptr(beta),
        fptr(running_mean), fptr(running_var), mean.data_ptr<float>(), invstd.data_ptr<float>(), scale.data_ptr<float>(),
        shift.data_ptr<float>());
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return {mean, invstd, scale, shift};
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> bn_coefficients(
    const at::Tensor& y, const c10::optional<at::Tensor>& gamma, const c10::optional<at::Tensor>& beta,
    const c10::optional<at::Tensor>& running_mean, const c10::optional<at::Tensor>& running_var, bool training,
    double momentum, double eps) {
    TORCH_CHECK(y.is_cuda() && y.is_contiguous(), "bn_coefficients: contiguous CUDA tensor required");
    const c10::cuda::CUDAGuard guard(y.device());
    const int C = (int)y.size(-1);
    TORCH_CHECK(C % 8 == 0 && C <= 4096, "bn_coefficients: C must be a multiple of 8 and <= 4096");
    const long long rows = y.numel() / C;
    auto fopt = y.options().dtype(at::kFloat);
    at::Tensor mean = at::empty({C}, fopt), invstd = at::empty({C}, fopt), scale = at::empty({C}, fopt), shift = at::empty({C}, fopt);
    auto fptr = [](const c10::optional<at::Tensor>& t) -> float* {
        if (!t.has_value() || !t->defined()) return nullptr;
        TORCH_CHECK(t->scalar_type() == at::kFloat && t->is_contiguous(), "BN parameters and buffers must be contiguous fp32");
        return t->data_ptr<float>();
    };
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    const int cb = (C + 127) / 128;
    if (training) {
        const int grid = stats_grid(rows);
        at::Tensor partial = at::empty({grid, 2, C}, fopt);
        SJ_BN_DISPATCH(y.scalar_type(), {
            bn_stats_partial_kernel<scalar_t><<<grid, kThreads, 2 * kThreads * 8 * sizeof(float), stream>>>(
                reinterpret_cast<const scalar_t*>(y.data_ptr()), rows, C, partial.data_ptr<float>());
        });
        C10_CUDA_KERNEL_LAUNCH_CHECK();
        bn_finalize_forward_kernel<<<(C + kFinCh - 1) / kFinCh, kFinCh * kFinSlices, 0, stream>>>(partial.data_ptr<float>(), grid, C, (double)rows, (float)eps,
                                                           (float)momentum, fptr(gamma), fptr(beta), fptr(running_mean),
                                                           fptr(running_var), mean.data_ptr<float>(), invstd.data_ptr<float>(),
                                                           scale.data_ptr<float>(), shift.data_ptr<float>());
    } else {
        TORCH_CHECK(fptr(running_mean) != nullptr && fptr(running_var) != nullptr, "frozen BN needs running statistics");
        bn_frozen_coeff_kernel<<<cb, 128, 0, stream>>>(C, (float)eps, fptr(gamma), fptr(beta), fptr(running_mean),
                                                       fptr(running_var), mean.data_ptr<float>(), invstd.data_ptr<float>(),
                                                       scale.data_ptr<float>(), shift.data_ptr<float>());
    }
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return {mean, invstd, scale, shift};
}

// spikes (+ residual) = LIF_T(y * scale + shift); y: [T, ..., C]; returns (out, ckpt | empty)
std::tuple<at::Tensor, at::Tensor> bn_lif_forward(const at::Tensor& y, const at::Tensor& scale, const at::Tensor& shift,
                                                  const c10::optional<at::Tensor>& residual, int64_t kind, double tau,
                                                  double v_th, double v_reset, bool soft_reset, double v_init,
                                                  bool save_ckpt) {
    TORCH_CHECK(y.is_cuda() && y.is_contiguous() && y.dim() >= 2, "bn_lif_forward: contiguous CUDA [T, ..., C] required");
    const c10::cuda::CUDAGuard guard(y.device());
    const int64_t T = y.size(0);
    const int C = (int)y.size(-1);
    const long long N = y.numel() / T;
    TORCH_CHECK(C % 8 == 0, "bn_lif_forward: C must be a multiple of 8");
    const ScanParams p = lif_params(T, N, kind, tau, v_th, v_reset, soft_reset, v_init);
    at::Tensor out = at::empty_like(y);
    const int n_ckpt = (int)((T + TCB - 1) / TCB) - 1;
    at::Tensor ckpt = (save_ckpt && n_ckpt > 0) ? at::empty({n_ckpt, N}, y.options().dtype(at::kFloat))
                                                 : at::empty({0}, y.options().dtype(at::kFloat));
    const void* res = nullptr;
    if (residual.has_value() && residual->defined()) {
        TORCH_CHECK(residual->is_contiguous() && residual->sizes() == y.sizes() && residual->scalar_type() == y.scalar_type(),
                    "bn_lif_forward: residual must match y");
        res = residual->data_ptr();
    }
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    SJ_BN_DISPATCH(y.scalar_type(), {
        constexpr int V = 16 / sizeof(scalar_t) > 8 ? 8 : 16 / sizeof(scalar_t);
        const unsigned grid = (unsigned)((N / V + kThreads - 1) / kThreads);
        SJ_BN_KIND(kind, {
            auto launch = [&](auto kern) {
                kern<<<grid, kThreads, 0, stream>>>(
                    p, C, reinterpret_cast<const scalar_t*>(y.data_ptr()), scale.data_ptr<float>(), shift.data_ptr<float>(),
                    reinterpret_cast<const scalar_t*>(res), reinterpret_cast<scalar_t*>(out.data_ptr()),
                    ckpt.numel() > 0 ? ckpt.data_ptr<float>() : nullptr);
            };
            if (T == TCB) {
                if (res != nullptr) launch(bn_lif_forward_kernel<scalar_t, V, KIND, TCB, true>);
                else launch(bn_lif_forward_kernel<scalar_t, V, KIND, TCB, false>);
            } else {
                if (res != nullptr) launch(bn_lif_forward_kernel<scalar_t, V, KIND, 0, true>);
                else launch(bn_lif_forward_kernel<scalar_t, V, KIND, 0, false>);
            }
        });
    });
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return {out, ckpt};
}

// returns (dy, grad_gamma, grad_beta)
std::tuple<at::Tensor, at::Tensor, at::Tensor> bn_lif_backward(
    const at::Tensor& g_out, const at::Tensor& y, const at::Tensor& scale, const at::Tensor& shift, const at::Tensor& mean,
    const at::Tensor& invstd, const c10::optional<at::Tensor>& gamma, const c10::optional<at::Tensor>& ckpt, bool training,
    int64_t kind, double tau, double v_th, double v_reset, bool soft_reset, double v_init, int64_t sg_id, double sg_p0,
    double sg_p1, bool detach_reset) {
    TORCH_CHECK(y.is_cuda() && y.is_contiguous(), "bn_lif_backward: contiguous CUDA tensor required");
    const c10::cuda::CUDAGuard guard(y.device());
    at::Tensor g = g_out.to(y.scalar_type()).contiguous();
    const int64_t T = y.size(0);
    const int C = (int)y.size(-1);
    const long long N = y.numel() / T;
    ScanParams p = lif_params(T, N, kind, tau, v_th, v_reset, soft_reset, v_init);
    p.sg_id = (int)sg_id; p.sg_p0 = (float)sg_p0; p.sg_p1 = (float)sg_p1; p.detach_reset = detach_reset ? 1 : 0;
    const int n_ckpt = (int)((T + TCB - 1) / TCB) - 1;
    const float* ck = nullptr;
    if (n_ckpt > 0) {
        TORCH_CHECK(ckpt.has_value() && ckpt->numel() == (int64_t)n_ckpt * N, "bn_lif_backward: missing checkpoints");
        ck = ckpt->data_ptr<float>();
    }
    auto fopt = y.options().dtype(at::kFloat);
    const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    at::Tensor gx = at::empty_like(y), dy = at::empty_like(y);
    at::Tensor grad_gamma = at::empty({C}, fopt), grad_beta = at::empty({C}, fopt);
    at::Tensor coef = at::empty({3, C}, fopt);
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    const float* gam = (gamma.has_value() && gamma->defined()) ? gamma->data_ptr<float>() : nullptr;
    SJ_BN_DISPATCH(y.scalar_type(), {
        constexpr int V = 16 / sizeof(scalar_t) > 8 ? 8 : 16 / sizeof(scalar_t);
        // pass 1 keeps a whole 4-step trajectory per element in registers: 4 elements per thread
        // (8-byte accesses for 16-bit types) leave room for three resident CTAs per SM
        constexpr int V1 = 4;
        const long long n_vec = N / V1;
        // gridDim * blockDim * V1 must be a multiple of C (see the kernel); m = C / gcd(C, blockDim * V1)
        long long gcd_a = C, gcd_b = (long long)kThreads * V1;
        while (gcd_b) { const long long t = gcd_a % gcd_b; gcd_a = gcd_b; gcd_b = t; }
        const long long m = C / gcd_a;
        // The grid is one wave of resident blocks (a grid-stride loop covers the rest): with more blocks than fit, the
        // last partial wave ran on half-empty SMs (1.5 waves measured: 444 blocks on 148 x 2 slots).
        // SJB200_BNLIF_OCC=3 selects the 80-register build (three CTAs per SM, 46 bytes of spills): measured equal or
        // slower than the 114-register build with two CTAs, which stays the default.
        static const int occ_choice = [] { const char* e = std::getenv("SJB200_BNLIF_OCC"); return e ? std::atoi(e) : 2; }();
        const int occ = (T == TCB && occ_choice == 3) ? 3 : 2;
        const long long want = std::max<long long>(1, std::min<long long>((n_vec + kThreads - 1) / kThreads, (long long)sms * occ));
        const int grid1 = (int)(std::max<long long>(1, want / m) * m);
        at::Tensor partial = at::empty({grid1, 2, C}, fopt);
        SJ_BN_KIND(kind, {
            auto launch = [&](auto kern) {
                kern<<<grid1, kThreads, kThreads * 2 * V1 * sizeof(float), stream>>>(
                    p, C, reinterpret_cast<const scalar_t*>(y.data_ptr()), reinterpret_cast<const scalar_t*>(g.data_ptr()),
                    scale.data_ptr<float>(), shift.data_ptr<float>(), ck,
                    reinterpret_cast<scalar_t*>(gx.data_ptr()), partial.data_ptr<float>());
            };
            if (T == TCB && occ == 3) launch(bn_lif_backward1_kernel<scalar_t, V1, KIND, TCB, 3>);     // 80 registers, three CTAs per SM
            else if (T == TCB) launch(bn_lif_backward1_kernel<scalar_t, V1, KIND, TCB, 2>);
            else launch(bn_lif_backward1_kernel<scalar_t, V1, KIND, 0>);
        });
        C10_CUDA_KERNEL_LAUNCH_CHECK();
        bn_finalize_backward_kernel<<<(C + kFinCh - 1) / kFinCh, kFinCh * kFinSlices, 0, stream>>>(
            partial.data_ptr<float>(), grid1, C, (double)(y.numel() / C), training ? 1 : 0, gam, mean.data_ptr<float>(),
            invstd.data_ptr<float>(), grad_gamma.data_ptr<float>(), grad_beta.data_ptr<float>(), coef.data_ptr<float>(),
            coef.data_ptr<float>() + C, coef.data_ptr<float>() + 2 * C);
        C10_CUDA_KERNEL_LAUNCH_CHECK();
        const long long total = y.numel();
        const unsigned grid2 = (unsigned)((total / V + kThreads - 1) / kThreads);
        bn_backward2_kernel<scalar_t, V><<<grid2, kThreads, 0, stream>>>(
            total, C, reinterpret_cast<const scalar_t*>(gx.data_ptr()), reinterpret_cast<const scalar_t*>(y.data_ptr()),
            coef.data_ptr<float>(), coef.data_ptr<float>() + C, coef.data_ptr<float>() + 2 * C,
            reinterpret_cast<scalar_t*>(dy.data_ptr()));
    });
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return {dy, grad_gamma, grad_beta};
}

}  // namespace sjb200

TORCH_LIBRARY_FRAGMENT(sjb200, m) {
    m.def("bn_coefficients(Tensor y, Tensor? gamma, Tensor? beta, Tensor(a!)? running_mean, Tensor(b!)? running_var, "
          "bool training, float momentum, float eps) -> (Tensor, Tensor, Tensor, Tensor)");
    m.def("bn_coefficients_partial(Tensor partial, int rows, Tensor? gamma, Tensor? beta, Tensor(a!)? running_mean, "
          "Tensor(b!)? running_var, float momentum, float eps) -> (Tensor, Tensor, Tensor, Tensor)");
    m.def("bn_lif_forward(Tensor y, Tensor scale, Tensor shift, Tensor? residual, int kind, float tau, float v_th, "
          "float v_reset, bool soft_reset, float v_init, bool save_ckpt) -> (Tensor, Tensor)");
    m.def("bn_lif_backward(Tensor g_out, Tensor y, Tensor scale, Tensor shift, Tensor mean, Tensor invstd, Tensor? gamma, "
          "Tensor? ckpt, bool training, int kind, float tau, float v_th, float v_reset, bool soft_reset, float v_init, "
          "int sg_id, float sg_p0, float sg_p1, bool detach_reset) -> (Tensor, Tensor, Tensor)");
}
TORCH_LIBRARY_IMPL(sjb200, CUDA, m) {
    m.impl("bn_coefficients", &sjb200::bn_coefficients);
    m.impl("bn_coefficients_partial", &sjb200::bn_coefficients_partial);
    m.impl("bn_lif_forward", &sjb200::bn_lif_forward);
    m.impl("bn_lif_backward", &sjb200::bn_lif_backward);
}
