// Patch matrix of a channels-last image batch for convolutions with very few input channels (the stems of the
// event-data and RGB networks: C_in = 2 or 3).  cuDNN pads such inputs to 8 channels and runs a generic kernel far
// below the memory rate; as a GEMM the stem is  Y[N*OH*OW, C_out] = A[N*OH*OW, KH*KW*C_in] . W^T  with a short K, and
// A is cheap to write because the image itself stays in L2.
//
//   x  [N, H, W, C]            16-bit, contiguous (channels last)
//   A  [N * OH * OW, Kp]       k = (kh * KW + kw) * C + c for k < KH * KW * C, zero for the padding columns up to Kp
//
// One thread writes eight consecutive k of one row at a time (one 16-byte store).
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "common.cuh"

namespace sjb200 {
namespace {

struct Im2colGeom { int N, H, W, C, OH, OW, KH, KW, sh, sw, ph, pw, K, Kp; };

// blockIdx.x = n * OH + oh: one block writes the OW * Kp elements of one output row of one image (contiguous in A) with
// 32-bit index arithmetic.  CFIX = 2: a pixel is one 32-bit word, so eight k are four word loads; CFIX = 0: any C.
template <typename T, int CFIX>
__global__ void __launch_bounds__(256)
im2col_nhwc_kernel(Im2colGeom g, const T* __restrict__ x, T* __restrict__ A) {
    const int C = CFIX > 0 ? CFIX : g.C;
    const int n = (int)blockIdx.x / g.OH, oh = (int)blockIdx.x - n * g.OH;
    const int ih0 = oh * g.sh - g.ph;
    const T* img = x + (size_t)n * g.H * g.W * C;
    T* arow = A + (size_t)blockIdx.x * g.OW * g.Kp;
    const int vpr = g.Kp / 8;
    const int n_pix = g.KH * g.KW;
    for (int v = threadIdx.x; v < g.OW * vpr; v += blockDim.x) {
        const int ow = v / vpr, k0 = (v - ow * vpr) * 8;
        const int iw0 = ow * g.sw - g.pw;
        if constexpr (CFIX == 2) {
            uint32_t w[4];
            int pk = k0 >> 1;
            int kh = pk / g.KW, kw = pk - kh * g.KW;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t val = 0;
                const int ih = ih0 + kh, iw = iw0 + kw;
                if (pk + j < n_pix && ih >= 0 && ih < g.H && iw >= 0 && iw < g.W)
                    val = *reinterpret_cast<const uint32_t*>(img + (ih * g.W + iw) * 2);
                w[j] = val;
                if (++kw == g.KW) { kw = 0; ++kh; }
            }
            *reinterpret_cast<uint4*>(arow + ow * g.Kp + k0) = make_uint4(w[0], w[1], w[2], w[3]);
        } else {
            Pack<T, 8> out;
            int c = k0 % C, kk = k0 / C;
            int kh = kk / g.KW, kw = kk - kh * g.KW;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                T val = from_f32<T>(0.0f);
                const int ih = ih0 + kh, iw = iw0 + kw;
                if (k0 + j < g.K && ih >= 0 && ih < g.H && iw >= 0 && iw < g.W) val = img[(ih * g.W + iw) * C + c];
                out.e[j] = val;
                if (++c == C) { c = 0; if (++kw == g.KW) { kw = 0; ++kh; } }
            }
            *reinterpret_cast<Pack<T, 8>*>(arow + ow * g.Kp + k0) = out;
        }
    }
}

}  // namespace

// x: [N, H, W, C] -> [N * OH * OW, Kp] with Kp = KH * KW * C rounded up to a multiple of 8
at::Tensor im2col_nhwc(const at::Tensor& x, int64_t KH, int64_t KW, int64_t sh, int64_t sw, int64_t ph, int64_t pw) {
    TORCH_CHECK(x.is_cuda() && x.dim() == 4 && x.is_contiguous(), "im2col_nhwc: contiguous CUDA [N, H, W, C] required");
    TORCH_CHECK(x.scalar_type() == at::kBFloat16 || x.scalar_type() == at::kHalf, "im2col_nhwc: bf16 or fp16 required");
    TORCH_CHECK(KH >= 1 && KW >= 1 && sh >= 1 && sw >= 1 && ph >= 0 && pw >= 0, "im2col_nhwc: bad window");
    Im2colGeom g{};
    g.N = (int)x.size(0); g.H = (int)x.size(1); g.W = (int)x.size(2); g.C = (int)x.size(3);
    g.KH = (int)KH; g.KW = (int)KW; g.sh = (int)sh; g.sw = (int)sw; g.ph = (int)ph; g.pw = (int)pw;
    TORCH_CHECK(g.H + 2 * g.ph >= g.KH && g.W + 2 * g.pw >= g.KW, "im2col_nhwc: window larger than the padded image");
    g.OH = (g.H + 2 * g.ph - g.KH) / g.sh + 1;
    g.OW = (g.W + 2 * g.pw - g.KW) / g.sw + 1;
    g.K = g.KH * g.KW * g.C;
    g.Kp = (g.K + 7) / 8 * 8;
    const c10::cuda::CUDAGuard guard(x.device());
    const long long rows = (long long)g.N * g.OH * g.OW;
    at::Tensor A = at::empty({rows, g.Kp}, x.options());
    if (rows == 0) return A;
    TORCH_CHECK((long long)g.H * g.W * g.C < 2147483647LL && (long long)g.OW * g.Kp < 2147483647LL, "im2col_nhwc: image too large for 32-bit indexing");
    const unsigned blocks = (unsigned)(g.N * g.OH);
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    if (x.scalar_type() == at::kBFloat16) {
        auto xp = reinterpret_cast<const __nv_bfloat16*>(x.data_ptr());
        auto ap = reinterpret_cast<__nv_bfloat16*>(A.data_ptr());
        if (g.C == 2) im2col_nhwc_kernel<__nv_bfloat16, 2><<<blocks, 256, 0, st>>>(g, xp, ap);
        else im2col_nhwc_kernel<__nv_bfloat16, 0><<<blocks, 256, 0, st>>>(g, xp, ap);
    } else {
        auto xp = reinterpret_cast<const __half*>(x.data_ptr());
        auto ap = reinterpret_cast<__half*>(A.data_ptr());
        if (g.C == 2) im2col_nhwc_kernel<__half, 2><<<blocks, 256, 0, st>>>(g, xp, ap);
        else im2col_nhwc_kernel<__half, 0><<<blocks, 256, 0, st>>>(g, xp, ap);
    }
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return A;
}

}  // namespace sjb200

TORCH_LIBRARY_FRAGMENT(sjb200, m) {
    m.def("im2col_nhwc(Tensor x, int KH, int KW, int sh, int sw, int ph, int pw) -> Tensor");
}
TORCH_LIBRARY_IMPL(sjb200, CUDA, m) {
    m.impl("im2col_nhwc", &sjb200::im2col_nhwc);
}
