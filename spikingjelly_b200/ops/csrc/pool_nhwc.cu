// MaxPool2d(kernel 3, stride 2, padding 1) on channels-last 16-bit feature maps (the stem of the spiking ResNets pools
// spike maps of [T * B, H, W, C]).
//
//   x    [N, H, W, C]     16-bit, contiguous (NHWC in memory)
//   out  [N, OH, OW, C]   window maximum; OH = (H - 1) / 2 + 1
//   idx  [N, OH, OW, C]   uint8: kh * 3 + kw of the first maximum in (kh, kw) scan order (PyTorch's tie rule)
//
// Forward: one thread per (pooled pixel, 8 channels), nine predicated 16-byte loads issued together.
// Backward: one thread per 2 x 2 input patch and 8 channels.  The patch (rows 2a, 2a + 1; columns 2b, 2b + 1) is covered
// by exactly the four windows (a .. a + 1) x (b .. b + 1): four (code, gradient) loads serve four input pixels, every
// input pixel is written exactly once (no atomics, no zero-fill pass), and the result is deterministic.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "common.cuh"

namespace sjb200 {
namespace {

constexpr int kThreads = 256;
constexpr int V = 8;

struct Geom { int N, H, W, C, OH, OW; };

template <typename T>
__global__ void __launch_bounds__(kThreads)
maxpool_forward_kernel(Geom g, const T* __restrict__ x, T* __restrict__ out, uint8_t* __restrict__ idx) {
    // blockIdx.x = n * OH + oh;  (blockIdx.y, threadIdx.x) = (ow, channel group)
    const int G = g.C / V;
    const int wc = (int)(blockIdx.y * blockDim.x + threadIdx.x);
    if (wc >= g.OW * G) return;
    const int ow = wc / G, c0 = (wc - ow * G) * V;
    const int n = (int)blockIdx.x / g.OH, oh = (int)blockIdx.x - n * g.OH;
    Pack<T, V> raw[9];
    bool have[9];
#pragma unroll
    for (int k = 0; k < 9; ++k) {
        const int ih = 2 * oh - 1 + k / 3, iw = 2 * ow - 1 + k % 3;
        have[k] = ih >= 0 && ih < g.H && iw >= 0 && iw < g.W;
        if (have[k]) raw[k] = load_raw_stream<T, V>(x + (((long long)n * g.H + ih) * g.W + iw) * g.C + c0);
    }
    float best[V];
    uint32_t code[V];
#pragma unroll
    for (int j = 0; j < V; ++j) { best[j] = -INFINITY; code[j] = 0; }
#pragma unroll
    for (int k = 0; k < 9; ++k) {
        if (!have[k]) continue;
        float v[V];
        unpack<T, V>(raw[k], v);
#pragma unroll
        for (int j = 0; j < V; ++j) {
            if (v[j] > best[j] || v[j] != v[j]) { best[j] = v[j]; code[j] = k; }     // NaN propagates, as in PyTorch
        }
    }
    const long long o = (((long long)n * g.OH + oh) * g.OW + ow) * g.C + c0;
    store_vec<T, V>(out + o, best);
    uint2 packed;
    packed.x = code[0] | (code[1] << 8) | (code[2] << 16) | (code[3] << 24);
    packed.y = code[4] | (code[5] << 8) | (code[6] << 16) | (code[7] << 24);
    *reinterpret_cast<uint2*>(idx + o) = packed;
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
maxpool_backward_kernel(Geom g, const T* __restrict__ gout, const uint8_t* __restrict__ idx, T* __restrict__ gx) {
    // blockIdx.x = n * PH + a;  (blockIdx.y, threadIdx.x) = (b, channel group)
    const int G = g.C / V;
    const int PH = (g.H + 1) / 2, PW = (g.W + 1) / 2;
    const int bc = (int)(blockIdx.y * blockDim.x + threadIdx.x);
    if (bc >= PW * G) return;
    const int pb = bc / G, c0 = (bc - pb * G) * V;
    const int n = (int)blockIdx.x / PH, pa = (int)blockIdx.x - n * PH;
    const int h0 = 2 * pa, w0 = 2 * pb;
    const bool row1 = h0 + 1 < g.H, col1 = w0 + 1 < g.W;
    uint2 code[4];
    Pack<T, V> graw[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int oh = pa + (k >> 1), ow = pb + (k & 1);
        code[k] = make_uint2(0xFFFFFFFFu, 0xFFFFFFFFu);       // no code is 0xFF: an absent window matches nothing
        if (oh < g.OH && ow < g.OW) {
            const long long o = (((long long)n * g.OH + oh) * g.OW + ow) * g.C + c0;
            code[k] = *reinterpret_cast<const uint2*>(idx + o);
            graw[k] = load_raw_stream<T, V>(gout + o);
        }
    }
    float gw[4][V];
#pragma unroll
    for (int k = 0; k < 4; ++k) unpack<T, V>(graw[k], gw[k]);
    const long long off00 = (((long long)n * g.H + h0) * g.W + w0) * g.C + c0;
    const long long rstride = (long long)g.W * g.C;
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
        store_vec<T, V>(gx + off00 + dh * rstride + dw * g.C, acc);
    }
}

Geom geom_of(const at::Tensor& x) {
    TORCH_CHECK(x.is_cuda() && x.dim() == 4 && x.is_contiguous(), "maxpool3x3s2_nhwc: contiguous CUDA [N, H, W, C] required");
    TORCH_CHECK(x.scalar_type() == at::kBFloat16 || x.scalar_type() == at::kHalf, "maxpool3x3s2_nhwc: bf16 or fp16 required");
    Geom g{};
    g.N = (int)x.size(0); g.H = (int)x.size(1); g.W = (int)x.size(2); g.C = (int)x.size(3);
    g.OH = (g.H - 1) / 2 + 1; g.OW = (g.W - 1) / 2 + 1;
    TORCH_CHECK(g.C % V == 0, "maxpool3x3s2_nhwc: C must be a multiple of 8");
    TORCH_CHECK((long long)g.N * ((g.H + 1) / 2) < 2147483647LL, "maxpool3x3s2_nhwc: too many rows for one grid");
    return g;
}

}  // namespace

std::tuple<at::Tensor, at::Tensor> maxpool3x3s2_nhwc_forward(const at::Tensor& x) {
    const Geom g = geom_of(x);
    const c10::cuda::CUDAGuard guard(x.device());
    at::Tensor out = at::empty({g.N, g.OH, g.OW, g.C}, x.options());
    at::Tensor idx = at::empty({g.N, g.OH, g.OW, g.C}, x.options().dtype(at::kByte));
    if (out.numel() == 0) return {out, idx};
    const dim3 grid((unsigned)(g.N * g.OH), (unsigned)((g.OW * (g.C / V) + kThreads - 1) / kThreads));
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    if (x.scalar_type() == at::kBFloat16)
        maxpool_forward_kernel<__nv_bfloat16><<<grid, kThreads, 0, st>>>(g, reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()),
                                                                         reinterpret_cast<__nv_bfloat16*>(out.data_ptr()), idx.data_ptr<uint8_t>());
    else
        maxpool_forward_kernel<__half><<<grid, kThreads, 0, st>>>(g, reinterpret_cast<const __half*>(x.data_ptr()),
                                                                  reinterpret_cast<__half*>(out.data_ptr()), idx.data_ptr<uint8_t>());
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return {out, idx};
}

// g_out, idx: [N, OH, OW, C];  returns dL/dx [N, H, W, C]
at::Tensor maxpool3x3s2_nhwc_backward(const at::Tensor& g_out, const at::Tensor& idx, int64_t H, int64_t W) {
    TORCH_CHECK(g_out.is_cuda() && g_out.dim() == 4 && g_out.is_contiguous() && idx.is_contiguous() && idx.sizes() == g_out.sizes() &&
                idx.scalar_type() == at::kByte, "maxpool3x3s2_nhwc_backward: contiguous [N, OH, OW, C] gradient and uint8 codes required");
    const c10::cuda::CUDAGuard guard(g_out.device());
    at::Tensor gx = at::empty({g_out.size(0), H, W, g_out.size(3)}, g_out.options());
    const Geom g = geom_of(gx);
    TORCH_CHECK(g.OH == g_out.size(1) && g.OW == g_out.size(2), "maxpool3x3s2_nhwc_backward: sizes do not match a 3x3 / 2 pooling of [H, W]");
    if (gx.numel() == 0) return gx;
    const dim3 grid((unsigned)(g.N * ((g.H + 1) / 2)), (unsigned)((((g.W + 1) / 2) * (g.C / V) + kThreads - 1) / kThreads));
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    if (g_out.scalar_type() == at::kBFloat16)
        maxpool_backward_kernel<__nv_bfloat16><<<grid, kThreads, 0, st>>>(g, reinterpret_cast<const __nv_bfloat16*>(g_out.data_ptr()),
                                                                          idx.data_ptr<uint8_t>(), reinterpret_cast<__nv_bfloat16*>(gx.data_ptr()));
    else
        maxpool_backward_kernel<__half><<<grid, kThreads, 0, st>>>(g, reinterpret_cast<const __half*>(g_out.data_ptr()),
                                                                   idx.data_ptr<uint8_t>(), reinterpret_cast<__half*>(gx.data_ptr()));
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return gx;
}

}  // namespace sjb200

TORCH_LIBRARY_FRAGMENT(sjb200, m) {
    m.def("maxpool3x3s2_nhwc_forward(Tensor x) -> (Tensor, Tensor)");
    m.def("maxpool3x3s2_nhwc_backward(Tensor g_out, Tensor idx, int H, int W) -> Tensor");
}
TORCH_LIBRARY_IMPL(sjb200, CUDA, m) {
    m.impl("maxpool3x3s2_nhwc_forward", &sjb200::maxpool3x3s2_nhwc_forward);
    m.impl("maxpool3x3s2_nhwc_backward", &sjb200::maxpool3x3s2_nhwc_backward);
}
