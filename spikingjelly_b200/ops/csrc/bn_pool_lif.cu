// BatchNorm -> MaxPool(3x3, stride 2, pad 1) -> multi-step LIF, fused, for NHWC feature maps
// (the Spikformer patch-splitting stem).  The normalised full-resolution map and the pooled map
// are never written: forward reads the convolution output once and writes spikes plus a one-byte
// argmax code per pooled element; backward routes gradients through that code.
//
//   y      [NB, H, W, C]   convolution output; NB = B when the input is the same at every time
//                           step ("static": pooled values are computed once and reused over T),
//                           else NB = T * B (time-major)
//   out    [T, B, OH, OW, C] spikes
//   idx    [NB, OH, OW, C]   kh * 3 + kw of the window maximum (first maximum wins, as in PyTorch)
//
// backward pass 1 (pooled resolution): BPTT; G = dL/d(pooled BN output) (summed over T when
//   static); per-channel sums of G and G * y_argmax as block partials;
// backward pass 2 (input resolution):  g = sum of G over the windows whose argmax is this pixel;
//   dy = A[c] g + B[c] y + D[c]  (BatchNorm backward in closed form).
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "bn_lif.h"
#include "neuron_scan.cuh"

namespace sjb200 {
namespace {

constexpr int kThreads = 256;
constexpr int V = 8;          // channels per thread (16 bytes of bf16 / fp16)
constexpr int kMaxT = 8;      // the backward keeps the whole trajectory in registers (template TMAX = 4 or 8)

struct PoolGeom {
    int B, T, H, W, C, OH, OW;
    int is_static;
};

template <typename T>
__device__ __forceinline__ void pooled_window(const T* __restrict__ y, const PoolGeom& g, int img, int oh, int ow, int c0,
                                              const float (&sc)[V], const float (&sh)[V], float (&best)[V],
                                              uint32_t (&code)[V]) {
#pragma unroll
    for (int j = 0; j < V; ++j) { best[j] = -INFINITY; code[j] = 0; }
#pragma unroll
    for (int kh = 0; kh < 3; ++kh) {
        const int ih = 2 * oh - 1 + kh;
        if (ih < 0 || ih >= g.H) continue;
#pragma unroll
        for (int kw = 0; kw < 3; ++kw) {
            const int iw = 2 * ow - 1 + kw;
            if (iw < 0 || iw >= g.W) continue;
            float v[V];
            load_vec<T, V>(y + (((long long)img * g.H + ih) * g.W + iw) * g.C + c0, v);
#pragma unroll
            for (int j = 0; j < V; ++j) {
                const float z = fmaf(v[j], sc[j], sh[j]);
                if (z > best[j]) { best[j] = z; code[j] = kh * 3 + kw; }
            }
        }
    }
}

// TFIX > 0: sequence length known at compile time; STATIC: one input image feeds every step.
template <typename T, int KIND, int TFIX, bool STATIC>
__global__ void __launch_bounds__(kThreads)
bn_pool_lif_forward_kernel(ScanParams p, PoolGeom g_in, const T* __restrict__ y, const float* __restrict__ scale,
                           const float* __restrict__ shift, T* __restrict__ out, uint8_t* __restrict__ idx) {
    PoolGeom g = g_in;
    g.is_static = STATIC ? 1 : 0;
    if constexpr (TFIX > 0) g.T = TFIX;
    const int G = g.C / V;
    const long long vec = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long n_vec = (long long)g.B * g.OH * g.OW * G;
    if (vec >= n_vec) return;
    const int cg = (int)(vec % G);
    long long pix = vec / G;
    const int ow = (int)(pix % g.OW); pix /= g.OW;
    const int oh = (int)(pix % g.OH);
    const int b = (int)(pix / g.OH);
    const int c0 = cg * V;
    const Neuron<KIND> nrn(p);
    float sc[V], sh[V], v[V], best[V];
    uint32_t code[V];
    load_vec<float, V>(scale + c0, sc);
    load_vec<float, V>(shift + c0, sh);
#pragma unroll
    for (int j = 0; j < V; ++j) v[j] = p.v_init_scalar;
    const long long per_step = (long long)g.B * g.OH * g.OW * g.C;
    const long long o_off = (((long long)b * g.OH + oh) * g.OW + ow) * g.C + c0;
#pragma unroll
    for (int t = 0; t < (TFIX > 0 ? TFIX : kMaxT); ++t) {
        if (t >= g.T) break;
        if (t == 0 || !g.is_static) {
            const int img = g.is_static ? b : t * g.B + b;
            pooled_window<T>(y, g, img, oh, ow, c0, sc, sh, best, code);
            uint2 packed;
            packed.x = code[0] | (code[1] << 8) | (code[2] << 16) | (code[3] << 24);
            packed.y = code[4] | (code[5] << 8) | (code[6] << 16) | (code[7] << 24);
            *reinterpret_cast<uint2*>(idx + (((long long)img * g.OH + oh) * g.OW + ow) * g.C + c0) = packed;
        }
        float s[V];
#pragma unroll
        for (int j = 0; j < V; ++j) {
            const float h = nrn.charge(best[j], v[j]);
            const bool f = nrn.fire(h);
            v[j] = nrn.reset(h, f);
            s[j] = f ? 1.0f : 0.0f;
        }
        store_vec<T, V>(out + (long long)t * per_step + o_off, s);
    }
}

// The host picks gridDim with (gridDim * blockDim) % (C / V) == 0, so a thread keeps its channel group.
// EXACT: T == TMAX (no per-step bounds predicates); STATIC: one input image feeds every step.
template <typename T, int KIND, int TMAX, bool EXACT, bool STATIC>
__global__ void __launch_bounds__(kThreads, 2)
bn_pool_lif_backward1_kernel(ScanParams p, PoolGeom g_in, const T* __restrict__ y, const uint8_t* __restrict__ idx,
                             const T* __restrict__ g_out, const float* __restrict__ scale,
                             const float* __restrict__ shift, T* __restrict__ Gout, float* __restrict__ partial) {
    extern __shared__ float s_buf[];   // [blockDim][2 V]
    PoolGeom g = g_in;
    g.is_static = STATIC ? 1 : 0;
    if constexpr (EXACT) g.T = TMAX;
    const int G = g.C / V;
    const long long n_vec = (long long)g.B * g.OH * g.OW * G;
    const long long first = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int cg = (int)(first % G);
    const int c0 = cg * V;
    const Neuron<KIND> nrn(p);
    const float dhdx = nrn.dh_dx(), dhdv = nrn.dh_dv(0.0f);
    const float kd = p.detach_reset ? 0.0f : 1.0f;
    const float k_s = p.soft_reset ? 0.0f : 1.0f;
    const float k_a = kd * (p.soft_reset ? -p.v_th : p.v_reset);
    const float k_b = kd * (p.soft_reset ? 0.0f : -1.0f);
    float sc[V], sh[V], a1[V], a2[V];
    load_vec<float, V>(scale + c0, sc);
    load_vec<float, V>(shift + c0, sh);
#pragma unroll
    for (int j = 0; j < V; ++j) { a1[j] = 0.0f; a2[j] = 0.0f; }
    const long long per_step = (long long)g.B * g.OH * g.OW * g.C;
    for (long long vec = first; vec < n_vec; vec += (long long)gridDim.x * blockDim.x) {
        long long pix = vec / G;
        const int ow = (int)(pix % g.OW); pix /= g.OW;
        const int oh = (int)(pix % g.OH);
        const int b = (int)(pix / g.OH);
        const long long o_off = (((long long)b * g.OH + oh) * g.OW + ow) * g.C + c0;
        // gather y at the argmax for every distinct pooled value
        float ya[TMAX][V];
#pragma unroll
        for (int t = 0; t < TMAX; ++t) {
            if (t < g.T && (t == 0 || !g.is_static)) {
                const int img = g.is_static ? b : t * g.B + b;
                const uint2 packed = *reinterpret_cast<const uint2*>(idx + (((long long)img * g.OH + oh) * g.OW + ow) * g.C + c0);
#pragma unroll
                for (int j = 0; j < V; ++j) {
                    const uint32_t code = ((j < 4 ? packed.x : packed.y) >> (8 * (j & 3))) & 0xFF;
                    const int ih = 2 * oh - 1 + (int)(code / 3), iw = 2 * ow - 1 + (int)(code % 3);
                    ya[t][j] = to_f32<T>(y[(((long long)img * g.H + ih) * g.W + iw) * g.C + c0 + j]);
                }
            }
        }
        // forward trajectory
        float h[TMAX][V];
        {
            float v[V];
#pragma unroll
            for (int j = 0; j < V; ++j) v[j] = p.v_init_scalar;
#pragma unroll
            for (int t = 0; t < TMAX; ++t) {
                if (t < g.T) {
#pragma unroll
                    for (int j = 0; j < V; ++j) {
                        const float x = fmaf(ya[g.is_static ? 0 : t][j], sc[j], sh[j]);
                        const float hh = nrn.charge(x, v[j]);
                        h[t][j] = hh;
                        v[j] = nrn.reset(hh, nrn.fire(hh));
                    }
                }
            }
        }
        // BPTT
        float c[V], Gs[V];
#pragma unroll
        for (int j = 0; j < V; ++j) { c[j] = 0.0f; Gs[j] = 0.0f; }
#pragma unroll
        for (int t = TMAX - 1; t >= 0; --t) {
            if (t < g.T) {
                float gs[V], sg[V], gx[V];
                load_vec_stream<T, V>(g_out + (long long)t * per_step + o_off, gs);
#pragma unroll
                for (int j = 0; j < V; ++j) sg[j] = h[t][j] - p.v_th;
                surrogate_grad_vec<V>(p.sg_id, sg, p.sg_p0, p.sg_p1);
#pragma unroll
                for (int j = 0; j < V; ++j) {
                    const float hh = h[t][j];
                    const float s = nrn.fire(hh) ? 1.0f : 0.0f;
                    const float dv_dh = fmaf(sg[j], fmaf(k_b, hh, k_a), fmaf(-k_s, s, 1.0f));
                    const float gh = fmaf(gs[j], sg[j], c[j] * dv_dh);
                    c[j] = gh * dhdv;
                    gx[j] = gh * dhdx;
                    Gs[j] += gx[j];
                }
                if (!g.is_static) {
                    const int img = t * g.B + b;
                    store_vec<T, V>(Gout + (((long long)img * g.OH + oh) * g.OW + ow) * g.C + c0, gx);
#pragma unroll
                    for (int j = 0; j < V; ++j) { a1[j] += gx[j]; a2[j] = fmaf(gx[j], ya[t][j], a2[j]); }
                }
            }
        }
        if (g.is_static) {
            store_vec<T, V>(Gout + o_off, Gs);
#pragma unroll
            for (int j = 0; j < V; ++j) { a1[j] += Gs[j]; a2[j] = fmaf(Gs[j], ya[0][j], a2[j]); }
        }
    }
#pragma unroll
    for (int j = 0; j < V; ++j) {
        s_buf[threadIdx.x * 2 * V + j] = a1[j];
        s_buf[threadIdx.x * 2 * V + V + j] = a2[j];
    }
    __syncthreads();
    const int g0 = (int)(((long long)blockIdx.x * blockDim.x) % G);
    float* outp = partial + (size_t)blockIdx.x * 2 * g.C;
    for (int i = threadIdx.x; i < 2 * g.C; i += blockDim.x) {
        const int which = i / g.C, ch = i % g.C;
        const int grp = ch / V, j = ch % V;
        const int f = ((grp - g0) % G + G) % G;
        float acc = 0.0f;
        for (int t = f; t < (int)blockDim.x; t += G) acc += s_buf[t * 2 * V + which * V + j];
        outp[i] = acc;
    }
}

// One thread owns a 2 x 2 patch of input pixels (rows 2a, 2a + 1; columns 2b, 2b + 1) and 8 channels.  The patch is
// covered by exactly the four windows (a .. a + 1) x (b .. b + 1), so four (argmax, gradient) loads serve four pixels,
// and every load of the thread (4 windows, 4 y vectors, 3 coefficient vectors) is issued before the first use:
// one memory round trip per thread instead of one per window.
template <typename T>
__global__ void __launch_bounds__(kThreads)
bn_pool_backward2_kernel(PoolGeom g, int NB, const T* __restrict__ y, const uint8_t* __restrict__ idx,
                         const T* __restrict__ Gin, const float* __restrict__ coefA, const float* __restrict__ coefB,
                         const float* __restrict__ coefD, T* __restrict__ dy) {
    // blockIdx.x = img * PH + a;  (blockIdx.y, threadIdx.x) = (b, channel group): 32-bit index arithmetic throughout
    const int G = g.C / V;
    const int PH = (g.H + 1) / 2, PW = (g.W + 1) / 2;
    const int bc = (int)(blockIdx.y * blockDim.x + threadIdx.x);
    if (bc >= PW * G) return;
    const int pb = bc / G, c0 = (bc - pb * G) * V;
    const int img = (int)blockIdx.x / PH, pa = (int)blockIdx.x - img * PH;
    const int h0 = 2 * pa, w0 = 2 * pb;
    const bool row1 = h0 + 1 < g.H, col1 = w0 + 1 < g.W;

    // windows: k = 2 * dh + dw -> (pa + dh, pb + dw)
    uint2 code[4];
    Pack<T, V> graw[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int oh = pa + (k >> 1), ow = pb + (k & 1);
        code[k] = make_uint2(0xFFFFFFFFu, 0xFFFFFFFFu);       // no argmax code is 0xFF: an absent window matches nothing
        if (oh < g.OH && ow < g.OW) {
            const long long o = (((long long)img * g.OH + oh) * g.OW + ow) * g.C + c0;
            code[k] = *reinterpret_cast<const uint2*>(idx + o);
            graw[k] = *reinterpret_cast<const Pack<T, V>*>(Gin + o);
        }
    }
    const long long off00 = (((long long)img * g.H + h0) * g.W + w0) * g.C + c0;
    const long long rstride = (long long)g.W * g.C;
    Pack<T, V> yraw[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        if (((k >> 1) == 0 || row1) && ((k & 1) == 0 || col1))
            yraw[k] = load_raw_stream<T, V>(y + off00 + (k >> 1) * rstride + (k & 1) * g.C);
    }
    float a[V], b[V], d[V];
    load_vec<float, V>(coefA + c0, a);
    load_vec<float, V>(coefB + c0, b);
    load_vec<float, V>(coefD + c0, d);

    float gw[4][V];
#pragma unroll
    for (int k = 0; k < 4; ++k) unpack<T, V>(graw[k], gw[k]);
    // pixel (dh, dw) of the patch lies at (kh, kw) = (1 + dh - 2 eh, 1 + dw - 2 ew) of window (eh, ew), eh <= dh, ew <= dw
#pragma unroll
    for (int px = 0; px < 4; ++px) {
        const int dh = px >> 1, dw = px & 1;
        if ((dh == 1 && !row1) || (dw == 1 && !col1)) continue;
        float acc[V];
#pragma unroll
        for (int j = 0; j < V; ++j) acc[j] = 0.0f;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int eh = k >> 1, ew = k & 1;
            if (eh > dh || ew > dw) continue;
            const uint32_t want = (uint32_t)((1 + dh - 2 * eh) * 3 + (1 + dw - 2 * ew));
#pragma unroll
            for (int j = 0; j < V; ++j) {
                const uint32_t cj = ((j < 4 ? code[k].x : code[k].y) >> (8 * (j & 3))) & 0xFF;
                acc[j] += (cj == want) ? gw[k][j] : 0.0f;
            }
        }
        float yy[V], o[V];
        unpack<T, V>(yraw[px], yy);
#pragma unroll
        for (int j = 0; j < V; ++j) o[j] = fmaf(a[j], acc[j], fmaf(b[j], yy[j], d[j]));
        store_vec<T, V>(dy + off00 + dh * rstride + dw * g.C, o);
    }
}

#define SJ_POOL_DISPATCH(DTYPE, ...)                                                        \
    switch (DTYPE) {                                                                         \
    case at::kHalf: { using scalar_t = __half; __VA_ARGS__; break; }                         \
    case at::kBFloat16: { using scalar_t = __nv_bfloat16; __VA_ARGS__; break; }              \
    default: TORCH_CHECK(false, "bn_pool_lif: bf16 or fp16 required, got ", DTYPE);          \
    }
#define SJ_POOL_KIND(KIND_VALUE, ...)                                                        \
    switch (KIND_VALUE) {                                                                    \
    case NK_IF: { constexpr int KIND = NK_IF; __VA_ARGS__; break; }                          \
    case NK_LIF_DI: { constexpr int KIND = NK_LIF_DI; __VA_ARGS__; break; }                  \
    case NK_LIF_NDI: { constexpr int KIND = NK_LIF_NDI; __VA_ARGS__; break; }                \
    default: TORCH_CHECK(false, "bn_pool_lif: neuron kind ", KIND_VALUE, " has no fused form"); \
    }

PoolGeom geom(const at::Tensor& y, int64_t T, bool is_static) {
    TORCH_CHECK(y.dim() == 4 && y.is_contiguous(), "bn_pool_lif: y must be a contiguous [NB, H, W, C] tensor");
    PoolGeom g{};
    const int NB = (int)y.size(0);
    g.T = (int)T; g.is_static = is_static ? 1 : 0;
    TORCH_CHECK(is_static || NB % T == 0, "bn_pool_lif: leading size must be T * B");
    g.B = is_static ? NB : NB / (int)T;
    g.H = (int)y.size(1); g.W = (int)y.size(2); g.C = (int)y.size(3);
    g.OH = (g.H - 1) / 2 + 1; g.OW = (g.W - 1) / 2 + 1;
    TORCH_CHECK(g.C % V == 0, "bn_pool_lif: C must be a multiple of 8");
    TORCH_CHECK(T >= 1 && T <= kMaxT, "bn_pool_lif: T must be in [1, ", kMaxT, "]");
    return g;
}

ScanParams lif_params(int64_t T, int64_t kind, double tau, double v_th, double v_reset, bool soft, double v_init) {
    ScanParams p{};
    p.T = (int)T; p.N = 0; p.kind = (int)kind; p.inv_tau = 1.0f / (float)tau;
    p.v_th = (float)v_th; p.v_reset = (float)v_reset; p.soft_reset = soft ? 1 : 0;
    p.v_init = nullptr; p.v_init_scalar = (float)v_init; p.r_ptr = nullptr;
    return p;
}

}  // namespace

// returns (spikes [T, B, OH, OW, C], idx [NB, OH, OW, C] uint8)
std::tuple<at::Tensor, at::Tensor> bn_pool_lif_forward(const at::Tensor& y, const at::Tensor& scale, const at::Tensor& shift,
                                                       int64_t T, bool is_static, int64_t kind, double tau, double v_th,
                                                       double v_reset, bool soft_reset, double v_init) {
    const c10::cuda::CUDAGuard guard(y.device());
    const PoolGeom g = geom(y, T, is_static);
    const ScanParams p = lif_params(T, kind, tau, v_th, v_reset, soft_reset, v_init);
    at::Tensor out = at::empty({T, g.B, g.OH, g.OW, g.C}, y.options());
    at::Tensor idx = at::empty({y.size(0), g.OH, g.OW, g.C}, y.options().dtype(at::kByte));
    const long long n_vec = (long long)g.B * g.OH * g.OW * (g.C / V);
    const unsigned grid = (unsigned)((n_vec + kThreads - 1) / kThreads);
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    SJ_POOL_DISPATCH(y.scalar_type(), {
        SJ_POOL_KIND(kind, {
            auto launch = [&](auto kern) {
                kern<<<grid, kThreads, 0, stream>>>(
                    p, g, reinterpret_cast<const scalar_t*>(y.data_ptr()), scale.data_ptr<float>(), shift.data_ptr<float>(),
                    reinterpret_cast<scalar_t*>(out.data_ptr()), idx.data_ptr<uint8_t>());
            };
            if (T == 4 && is_static) launch(bn_pool_lif_forward_kernel<scalar_t, KIND, 4, true>);
            else if (T == 4) launch(bn_pool_lif_forward_kernel<scalar_t, KIND, 4, false>);
            else if (is_static) launch(bn_pool_lif_forward_kernel<scalar_t, KIND, 0, true>);
            else launch(bn_pool_lif_forward_kernel<scalar_t, KIND, 0, false>);
        });
    });
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return {out, idx};
}

// returns (dy [NB, H, W, C], grad_gamma, grad_beta)
std::tuple<at::Tensor, at::Tensor, at::Tensor> bn_pool_lif_backward(
    const at::Tensor& g_out, const at::Tensor& y, const at::Tensor& idx, const at::Tensor& scale, const at::Tensor& shift,
    const at::Tensor& mean, const at::Tensor& invstd, const c10::optional<at::Tensor>& gamma, bool training, int64_t T,
    bool is_static, int64_t kind, double tau, double v_th, double v_reset, bool soft_reset, double v_init, int64_t sg_id,
    double sg_p0, double sg_p1, bool detach_reset) {
    const c10::cuda::CUDAGuard guard(y.device());
    const PoolGeom g = geom(y, T, is_static);
    ScanParams p = lif_params(T, kind, tau, v_th, v_reset, soft_reset, v_init);
    p.sg_id = (int)sg_id; p.sg_p0 = (float)sg_p0; p.sg_p1 = (float)sg_p1; p.detach_reset = detach_reset ? 1 : 0;
    at::Tensor go = g_out.to(y.scalar_type()).contiguous();
    auto fopt = y.options().dtype(at::kFloat);
    const int NB = (int)y.size(0);
    at::Tensor Gt = at::empty({NB, g.OH, g.OW, g.C}, y.options());
    at::Tensor dy = at::empty_like(y);
    at::Tensor grad_gamma = at::empty({g.C}, fopt), grad_beta = at::empty({g.C}, fopt), coef = at::empty({3, g.C}, fopt);
    const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    const int G = g.C / V;
    const long long n_vec = (long long)g.B * g.OH * g.OW * G;
    // (grid * blockDim) % G == 0
    long long ga = G, gb = kThreads;
    while (gb) { const long long t = ga % gb; ga = gb; gb = t; }
    const long long m = G / ga;
    const long long want = std::max<long long>(1, std::min<long long>((n_vec + kThreads - 1) / kThreads, (long long)sms * 2));
    const int grid1 = (int)(std::max<long long>(1, want / m) * m);
    at::Tensor partial = at::empty({grid1, 2, g.C}, fopt);
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    const float* gam = (gamma.has_value() && gamma->defined()) ? gamma->data_ptr<float>() : nullptr;
    SJ_POOL_DISPATCH(y.scalar_type(), {
        SJ_POOL_KIND(kind, {
            auto launch = [&](auto kern) {
                kern<<<grid1, kThreads, kThreads * 2 * V * sizeof(float), stream>>>(
                    p, g, reinterpret_cast<const scalar_t*>(y.data_ptr()), idx.data_ptr<uint8_t>(),
                    reinterpret_cast<const scalar_t*>(go.data_ptr()), scale.data_ptr<float>(), shift.data_ptr<float>(),
                    reinterpret_cast<scalar_t*>(Gt.data_ptr()), partial.data_ptr<float>());
            };
            if (T == 4) {
                if (is_static) launch(bn_pool_lif_backward1_kernel<scalar_t, KIND, 4, true, true>);
                else launch(bn_pool_lif_backward1_kernel<scalar_t, KIND, 4, true, false>);
            } else if (T < 4) {
                if (is_static) launch(bn_pool_lif_backward1_kernel<scalar_t, KIND, 4, false, true>);
                else launch(bn_pool_lif_backward1_kernel<scalar_t, KIND, 4, false, false>);
            } else {
                if (is_static) launch(bn_pool_lif_backward1_kernel<scalar_t, KIND, 8, false, true>);
                else launch(bn_pool_lif_backward1_kernel<scalar_t, KIND, 8, false, false>);
            }
        });
    });
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    launch_bn_finalize_backward(partial.data_ptr<float>(), grid1, g.C, (double)(y.numel() / g.C), training ? 1 : 0, gam,
                                mean.data_ptr<float>(), invstd.data_ptr<float>(), grad_gamma.data_ptr<float>(),
                                grad_beta.data_ptr<float>(), coef.data_ptr<float>(), coef.data_ptr<float>() + g.C,
                                coef.data_ptr<float>() + 2 * g.C, stream);
    const dim3 grid2((unsigned)(NB * ((g.H + 1) / 2)), (unsigned)((((g.W + 1) / 2) * G + kThreads - 1) / kThreads));
    SJ_POOL_DISPATCH(y.scalar_type(), {
        bn_pool_backward2_kernel<scalar_t><<<grid2, kThreads, 0, stream>>>(
            g, NB, reinterpret_cast<const scalar_t*>(y.data_ptr()), idx.data_ptr<uint8_t>(),
            reinterpret_cast<const scalar_t*>(Gt.data_ptr()), coef.data_ptr<float>(), coef.data_ptr<float>() + g.C,
            coef.data_ptr<float>() + 2 * g.C, reinterpret_cast<scalar_t*>(dy.data_ptr()));
    });
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return {dy, grad_gamma, grad_beta};
}

}  // namespace sjb200

TORCH_LIBRARY_FRAGMENT(sjb200, m) {
    m.def("bn_pool_lif_forward(Tensor y, Tensor scale, Tensor shift, int T, bool is_static, int kind, float tau, float v_th, "
          "float v_reset, bool soft_reset, float v_init) -> (Tensor, Tensor)");
    m.def("bn_pool_lif_backward(Tensor g_out, Tensor y, Tensor idx, Tensor scale, Tensor shift, Tensor mean, Tensor invstd, "
          "Tensor? gamma, bool training, int T, bool is_static, int kind, float tau, float v_th, float v_reset, "
          "bool soft_reset, float v_init, int sg_id, float sg_p0, float sg_p1, bool detach_reset) -> (Tensor, Tensor, Tensor)");
}
TORCH_LIBRARY_IMPL(sjb200, CUDA, m) {
    m.impl("bn_pool_lif_forward", &sjb200::bn_pool_lif_forward);
    m.impl("bn_pool_lif_backward", &sjb200::bn_pool_lif_backward);
}
