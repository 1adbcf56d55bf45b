// Implicit-GEMM 2-D convolution on the 5th-generation tensor cores: forward, data gradient and weight gradient of a
// channels-last (NHWC) convolution run in the persistent TMA / tcgen05 / TMEM kernel of gemm_tcgen05_kernel.cuh.  The
// patch matrix is never materialised: the TMA unit gathers it (im2col tensor maps, one load = 128 or 64 pixels x 64
// channels of one filter tap, zero-filled outside the image) straight into the 128-byte-swizzled operand tiles.
//
//   forward   y[(n, oh, ow), k]  = sum_{r, s, c} x[n, oh*sh - ph + r*dh, ow*sw - pw + s*dw, c] * w[k, r, s, c]
//             A = x gathered (K-major rows of 64 channels), B = w as [Cout][R*S*C] (K-major), D = NHWC output rows;
//             the epilogue can emit the per-channel sums a following batch norm needs.
//   dgrad     dx[n, h, w, c]     = sum_{r, s, k} dy[n, (h + ph - r) / sh, (w + pw - s) / sw, k] * w[k, r, s, c]
//             (terms with a non-integer position vanish).  One launch per parity class (h mod sh, w mod sw): within a
//             class the contributing taps are r = r0 + sh*t, the gathered tensor is dy walked with unit stride, B is the
//             SAME filter tensor read MN-major (rows = Cout) at the tap's column offset, and rows are scattered to the
//             class's pixels.  Stride 1 is the single-class case with a dense (TMA-stored) result.
//   wgrad     dw[k, (r, s, c)]   = sum_{pixels} dy[pixel, k] * x_gathered[pixel, (r, s, c)]
//             A = dy (MN-major), B = x gathered 64 pixels at a time (MN-major), contraction over all output pixels with
//             split-K and a fixed-order fp32 reduction.
//
// Filters are passed as [Cout, R, S, Cin] (the memory of a channels-last [Cout, Cin, R, S] tensor).  Channel counts
// must be multiples of 64 (one 128-byte swizzle row of 16-bit channels per pixel and tap); other layers stay with the
// callers' fallbacks.
#include "gemm_tcgen05_kernel.cuh"

namespace sjb200 {
using namespace tc;

namespace {

using EncodeIm2colFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const int*, const int*, cuuint32_t, cuuint32_t, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeIm2colFn encode_im2col_fn() {
    static EncodeIm2colFn fn = []() -> EncodeIm2colFn {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &p, cudaEnableDefault, &q);
        TORCH_CHECK(e == cudaSuccess && q == cudaDriverEntryPointSuccess && p != nullptr,
                    "cuTensorMapEncodeIm2col is not available from the driver");
        return reinterpret_cast<EncodeIm2colFn>(p);
    }();
    return fn;
}

// im2col map over a contiguous NHWC 16-bit tensor.  The bounding box of start positions is
// [lower, extent + upper) per spatial axis, walked with `step`; one load gathers `pixels` positions x 64 channels.
CUtensorMap make_im2col_map(const void* base, int64_t Nb, int64_t H, int64_t W, int64_t C, int lower_h, int lower_w, int upper_h,
                            int upper_w, int step_h, int step_w, int pixels, bool bf16) {
    TORCH_CHECK(reinterpret_cast<uintptr_t>(base) % 16 == 0, "conv: tensor base must be 16-byte aligned");
    TORCH_CHECK(C % 64 == 0, "conv: channels must be a multiple of 64");
    TORCH_CHECK(lower_h >= -128 && lower_h <= 127 && lower_w >= -128 && lower_w <= 127 && upper_h >= -128 && upper_h <= 127 &&
                upper_w >= -128 && upper_w <= 127, "conv: padding / filter extent outside the im2col corner range");
    TORCH_CHECK(step_h >= 1 && step_h <= 8 && step_w >= 1 && step_w <= 8, "conv: stride must be in [1, 8]");
    TORCH_CHECK(H + upper_h - lower_h > 0 && W + upper_w - lower_w > 0, "conv: empty traversal box");
    CUtensorMap m;
    cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)Nb};
    cuuint64_t strides[3] = {(cuuint64_t)C * 2, (cuuint64_t)W * C * 2, (cuuint64_t)H * W * C * 2};
    int lower[2] = {lower_w, lower_h};                   // same order as the dimensions: W, then H
    int upper[2] = {upper_w, upper_h};
    cuuint32_t estr[4] = {1u, (cuuint32_t)step_w, (cuuint32_t)step_h, 1u};
    CUresult r = encode_im2col_fn()(&m, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                                    const_cast<void*>(base), dims, strides, lower, upper, 64u, (cuuint32_t)pixels, estr,
                                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeIm2col failed with code ", (int)r);
    return m;
}

int64_t out_extent(int64_t in, int64_t pad, int64_t k, int64_t dil, int64_t stride) {
    return (in + 2 * pad - dil * (k - 1) - 1) / stride + 1;
}

void check_nhwc(const at::Tensor& t, const char* what) {
    TORCH_CHECK(t.is_cuda() && t.dim() == 4 && t.is_contiguous(), "conv: ", what, " must be a contiguous 4-D CUDA tensor (NHWC / KRSC)");
    TORCH_CHECK(t.scalar_type() == at::kBFloat16 || t.scalar_type() == at::kHalf, "conv: ", what, " must be bf16 or fp16");
}

struct ConvShape {
    int64_t Nb, H, W, C, K, R, S, Ho, Wo;
    int sh, sw, ph, pw, dh, dw;
};

ConvShape make_shape(int64_t Nb, int64_t H, int64_t W, int64_t C, const at::Tensor& w, at::IntArrayRef stride, at::IntArrayRef padding,
                     at::IntArrayRef dilation) {
    TORCH_CHECK(stride.size() == 2 && padding.size() == 2 && dilation.size() == 2, "conv: stride, padding, dilation take two values");
    ConvShape s{};
    s.Nb = Nb; s.H = H; s.W = W; s.C = C;
    s.K = w.size(0); s.R = w.size(1); s.S = w.size(2);
    TORCH_CHECK(w.size(3) == C, "conv: filter has ", w.size(3), " input channels, the activation ", C);
    s.sh = (int)stride[0]; s.sw = (int)stride[1]; s.ph = (int)padding[0]; s.pw = (int)padding[1];
    s.dh = (int)dilation[0]; s.dw = (int)dilation[1];
    s.Ho = out_extent(H, s.ph, s.R, s.dh, s.sh);
    s.Wo = out_extent(W, s.pw, s.S, s.dw, s.sw);
    TORCH_CHECK(s.Ho > 0 && s.Wo > 0, "conv: empty output");
    TORCH_CHECK(C % 64 == 0 && s.K % 64 == 0, "conv: channel counts must be multiples of 64 (got ", C, " -> ", s.K, ")");
    TORCH_CHECK(Nb * s.Ho * s.Wo < (int64_t)1 << 31 && Nb * H * W < (int64_t)1 << 31, "conv: more than 2^31 pixels");
    return s;
}

}  // namespace

// y rows [Nb*Ho*Wo, Cout] (= NHWC output) and, if want_stats, the batch-norm partial sums of gemm_16bit_stats.
std::tuple<at::Tensor, at::Tensor> conv2d_nhwc_forward(const at::Tensor& x, const at::Tensor& w, at::IntArrayRef stride,
                                                        at::IntArrayRef padding, at::IntArrayRef dilation, bool want_stats) {
    check_nhwc(x, "input");
    check_nhwc(w, "filter");
    TORCH_CHECK(x.scalar_type() == w.scalar_type(), "conv: input and filter dtypes differ");
    const c10::cuda::CUDAGuard guard(x.device());
    C10_CUDA_CHECK(cudaFree(nullptr));
    const ConvShape s = make_shape(x.size(0), x.size(1), x.size(2), x.size(3), w, stride, padding, dilation);
    const bool bf16 = x.scalar_type() == at::kBFloat16;
    const int64_t M = s.Nb * s.Ho * s.Wo, N = s.K, K = s.R * s.S * s.C;
    const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    const int BN = N > 128 ? 256 : (N > 64 ? 128 : 64);
    const int tiles = (int)(((M + BM - 1) / BM) * ((N + BN - 1) / BN));

    GemmArgs g{};
    g.M = (int)M; g.N = (int)N; g.K = (int)K; g.ldd = (int)N;
    g.split_k = 1; g.kb_per_split = (int)(K / BK);
    g.out_f32 = 0; g.ab_format = bf16 ? 1 : 0; g.out_bf16 = bf16 ? 1 : 0;
    at::Tensor out = at::empty({M, N}, x.options());
    at::Tensor stats = at::empty({0}, x.options().dtype(at::kFloat));
    if (want_stats) {
        stats = at::empty({(M + BM - 1) / BM * 4, 2, N}, x.options().dtype(at::kFloat));
        g.stats = stats.data_ptr<float>();
    }
    ConvGeom cg{};
    cg.Ht = (int)s.Ho; cg.Wt = (int)s.Wo; cg.base_h = -s.ph; cg.base_w = -s.pw; cg.step_h = s.sh; cg.step_w = s.sw;
    cg.taps_h = (int)s.R; cg.taps_w = (int)s.S; cg.dil_h = s.dh; cg.dil_w = s.dw;
    cg.CA = (int)s.C; cg.CN = (int)s.C;
    cg.wr0 = 0; cg.wr_step = 1; cg.ws0 = 0; cg.ws_step = 1; cg.S = (int)s.S;
    const CUtensorMap ta = make_im2col_map(x.data_ptr(), s.Nb, s.H, s.W, s.C, -s.ph, -s.pw, s.ph - s.dh * ((int)s.R - 1),
                                           s.pw - s.dw * ((int)s.S - 1), s.sh, s.sw, BM, bf16);
    const CUtensorMap tb = make_map(w.data_ptr(), N, K, K, BN, bf16);
    const CUtensorMap td = make_map(out.data_ptr(), M, N, N, 32, bf16, 32);
    KernelStatus* stp = reinterpret_cast<KernelStatus*>(status_word(x.device()).data_ptr<int>());
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    const int grid = std::min(tiles, sms);
    if (BN == 256) launch<256, 4, false, false, 2, 1>(ta, tb, td, out.data_ptr(), g, stp, grid, stream, cg);
    else if (BN == 128) launch<128, 6, false, false, 2, 1>(ta, tb, td, out.data_ptr(), g, stp, grid, stream, cg);
    else launch<64, 8, false, false, 2, 1>(ta, tb, td, out.data_ptr(), g, stp, grid, stream, cg);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return {out, stats};
}

// dx [Nb, H, W, Cin] from dy rows [Nb*Ho*Wo, Cout] (NHWC) and the forward filter [Cout, R, S, Cin].  Dilation 1 only.
at::Tensor conv2d_nhwc_dgrad(const at::Tensor& gy, const at::Tensor& w, int64_t H, int64_t W, at::IntArrayRef stride,
                             at::IntArrayRef padding) {
    check_nhwc(w, "filter");
    TORCH_CHECK(gy.is_cuda() && gy.is_contiguous() && gy.scalar_type() == w.scalar_type(), "conv dgrad: contiguous output gradient of the filter's dtype required");
    const c10::cuda::CUDAGuard guard(gy.device());
    C10_CUDA_CHECK(cudaFree(nullptr));
    const int64_t one[2] = {1, 1};
    const int64_t Cout = w.size(0), Cin = w.size(3);
    ConvShape s{};
    {
        // shapes of the forward convolution
        const int64_t sh = stride[0], sw = stride[1], ph = padding[0], pw = padding[1];
        const int64_t Ho = out_extent(H, ph, w.size(1), 1, sh), Wo = out_extent(W, pw, w.size(2), 1, sw);
        TORCH_CHECK(gy.numel() % (Ho * Wo * Cout) == 0, "conv dgrad: output gradient does not match the forward shape");
        s = make_shape(gy.numel() / (Ho * Wo * Cout), H, W, Cin, w, stride, padding, at::IntArrayRef(one, 2));
    }
    const bool bf16 = gy.scalar_type() == at::kBFloat16;
    const bool dense = s.sh == 1 && s.sw == 1;
    bool every_class_has_taps = true;
    for (int a = 0; a < s.sh; ++a) if ((a + s.ph) % s.sh >= s.R) every_class_has_taps = false;
    for (int b = 0; b < s.sw; ++b) if ((b + s.pw) % s.sw >= s.S) every_class_has_taps = false;
    at::Tensor gx = every_class_has_taps ? at::empty({s.Nb, H, W, Cin}, gy.options()) : at::zeros({s.Nb, H, W, Cin}, gy.options());
    const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    KernelStatus* stp = reinterpret_cast<KernelStatus*>(status_word(gy.device()).data_ptr<int>());
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    const int64_t N = Cin;
    const int BN = N > 128 ? 256 : (N > 64 ? 128 : 64);
    // the filter as a [Cout, R*S*Cin] matrix read MN-major: boxes of 64 output channels (k) x 64 input channels
    const CUtensorMap tb = make_map(w.data_ptr(), Cout, s.R * s.S * Cin, s.R * s.S * Cin, BK, bf16);

    for (int a = 0; a < s.sh; ++a) {
        const int64_t cnt_h = (H - a + s.sh - 1) / s.sh;
        const int r0 = (a + s.ph) % s.sh;
        if (cnt_h <= 0 || r0 >= s.R) continue;
        const int nt_h = ((int)s.R - r0 + s.sh - 1) / s.sh;
        const int q_h = (a + s.ph - r0) / s.sh;
        for (int b = 0; b < s.sw; ++b) {
            const int64_t cnt_w = (W - b + s.sw - 1) / s.sw;
            const int s0 = (b + s.pw) % s.sw;
            if (cnt_w <= 0 || s0 >= s.S) continue;
            const int nt_w = ((int)s.S - s0 + s.sw - 1) / s.sw;
            const int q_w = (b + s.pw - s0) / s.sw;
            const int64_t M = s.Nb * cnt_h * cnt_w, K = (int64_t)nt_h * nt_w * Cout;
            const int tiles = (int)(((M + BM - 1) / BM) * ((N + BN - 1) / BN));
            GemmArgs g{};
            g.M = (int)M; g.N = (int)N; g.K = (int)K; g.ldd = (int)N;
            g.split_k = 1; g.kb_per_split = (int)(K / BK);
            g.out_f32 = 0; g.ab_format = bf16 ? 1 : 0; g.out_bf16 = bf16 ? 1 : 0;
            ConvGeom cg{};
            cg.Ht = (int)cnt_h; cg.Wt = (int)cnt_w;
            cg.base_h = q_h - (nt_h - 1); cg.base_w = q_w - (nt_w - 1); cg.step_h = 1; cg.step_w = 1;
            cg.taps_h = nt_h; cg.taps_w = nt_w; cg.dil_h = 1; cg.dil_w = 1;
            cg.CA = (int)Cout; cg.CN = (int)Cin;
            cg.wr0 = r0 + s.sh * (nt_h - 1); cg.wr_step = -s.sh; cg.ws0 = s0 + s.sw * (nt_w - 1); cg.ws_step = -s.sw; cg.S = (int)s.S;
            cg.scatter = dense ? 0 : 1; cg.out_H = (int)H; cg.out_W = (int)W;
            cg.out_mul_h = s.sh; cg.out_mul_w = s.sw; cg.out_add_h = a; cg.out_add_w = b;
            const CUtensorMap ta = make_im2col_map(gy.data_ptr(), s.Nb, s.Ho, s.Wo, Cout, cg.base_h, cg.base_w,
                                                   (int)(cnt_h + cg.base_h - s.Ho), (int)(cnt_w + cg.base_w - s.Wo), 1, 1, BM, bf16);
            const CUtensorMap td = dense ? make_map(gx.data_ptr(), M, N, N, 32, bf16, 32) : ta;
            const int grid = std::min(tiles, sms);
            if (BN == 256) launch<256, 4, false, true, 2, 1>(ta, tb, td, gx.data_ptr(), g, stp, grid, stream, cg);
            else if (BN == 128) launch<128, 6, false, true, 2, 1>(ta, tb, td, gx.data_ptr(), g, stp, grid, stream, cg);
            else launch<64, 8, false, true, 2, 1>(ta, tb, td, gx.data_ptr(), g, stp, grid, stream, cg);
            C10_CUDA_KERNEL_LAUNCH_CHECK();
        }
    }
    return gx;
}

// dw [Cout, R, S, Cin] (fp32) from x [Nb, H, W, Cin] and dy rows [Nb*Ho*Wo, Cout].
at::Tensor conv2d_nhwc_wgrad(const at::Tensor& x, const at::Tensor& gy, int64_t R, int64_t S, at::IntArrayRef stride,
                             at::IntArrayRef padding, at::IntArrayRef dilation) {
    check_nhwc(x, "input");
    TORCH_CHECK(gy.is_cuda() && gy.is_contiguous() && gy.scalar_type() == x.scalar_type(), "conv wgrad: contiguous output gradient of the input's dtype required");
    const c10::cuda::CUDAGuard guard(x.device());
    C10_CUDA_CHECK(cudaFree(nullptr));
    const int64_t Nb = x.size(0), H = x.size(1), W = x.size(2), Cin = x.size(3);
    const int sh = (int)stride[0], sw = (int)stride[1], ph = (int)padding[0], pw = (int)padding[1], dh = (int)dilation[0], dw = (int)dilation[1];
    const int64_t Ho = out_extent(H, ph, R, dh, sh), Wo = out_extent(W, pw, S, dw, sw);
    const int64_t P = Nb * Ho * Wo;
    TORCH_CHECK(Ho > 0 && Wo > 0 && gy.numel() % P == 0, "conv wgrad: output gradient does not match the forward shape");
    const int64_t Cout = gy.numel() / P;
    TORCH_CHECK(Cin % 64 == 0 && Cout % 64 == 0, "conv: channel counts must be multiples of 64");
    TORCH_CHECK(P < (int64_t)1 << 31, "conv: more than 2^31 pixels");
    const bool bf16 = x.scalar_type() == at::kBFloat16;
    const int64_t M = Cout, N = R * S * Cin, K = P;
    const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    const int BN = 256;
    const int tiles = (int)(((M + BM - 1) / BM) * ((N + BN - 1) / BN));
    const int kb_total = (int)((K + BK - 1) / BK);
    int splits = std::max(1, std::min(sms / std::max(tiles, 1), kb_total / 4));
    if (tiles >= sms) splits = 1;
    int kb_per = (kb_total + splits - 1) / splits;
    splits = (kb_total + kb_per - 1) / kb_per;

    GemmArgs g{};
    g.M = (int)M; g.N = (int)N; g.K = (int)K; g.ldd = (int)N;
    g.split_k = splits; g.kb_per_split = kb_per;
    g.out_f32 = 1; g.ab_format = bf16 ? 1 : 0; g.out_bf16 = bf16 ? 1 : 0;
    ConvGeom cg{};
    cg.Ht = (int)Ho; cg.Wt = (int)Wo; cg.base_h = -ph; cg.base_w = -pw; cg.step_h = sh; cg.step_w = sw;
    cg.taps_h = (int)R; cg.taps_w = (int)S; cg.dil_h = dh; cg.dil_w = dw;
    cg.CA = (int)Cin; cg.CN = (int)Cin; cg.S = (int)S;
    // A: dy as [pixels, Cout], MN-major boxes of 64 pixels x 64 output channels
    const CUtensorMap ta = make_map(gy.data_ptr(), P, Cout, Cout, BK, bf16);
    const CUtensorMap tb = make_im2col_map(x.data_ptr(), Nb, H, W, Cin, -ph, -pw, ph - dh * ((int)R - 1), pw - dw * ((int)S - 1), sh, sw,
                                           BK, bf16);
    at::Tensor out = at::empty({Cout, R, S, Cin}, x.options().dtype(at::kFloat));
    at::Tensor scratch;
    void* dptr = out.data_ptr();
    if (splits > 1) {
        scratch = at::empty({splits, M, N}, x.options().dtype(at::kFloat));
        dptr = scratch.data_ptr();
    }
    KernelStatus* stp = reinterpret_cast<KernelStatus*>(status_word(x.device()).data_ptr<int>());
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    const int grid = std::min(tiles * splits, sms);
    launch<256, 4, true, true, 2, 2>(ta, tb, ta, dptr, g, stp, grid, stream, cg);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    if (splits > 1) {
        const long long mn = (long long)M * N;
        const unsigned blocks = (unsigned)((mn / 4 + 256) / 256);
        splitk_reduce_kernel<float><<<blocks, 256, 0, stream>>>(scratch.data_ptr<float>(), out.data_ptr<float>(), mn, splits, 0.f, nullptr);
        C10_CUDA_KERNEL_LAUNCH_CHECK();
    }
    return out;
}

}  // namespace sjb200

TORCH_LIBRARY_FRAGMENT(sjb200, m) {
    m.def("conv2d_nhwc_forward(Tensor x, Tensor w, int[] stride, int[] padding, int[] dilation, bool want_stats) -> (Tensor, Tensor)");
    m.def("conv2d_nhwc_dgrad(Tensor gy, Tensor w, int H, int W, int[] stride, int[] padding) -> Tensor");
    m.def("conv2d_nhwc_wgrad(Tensor x, Tensor gy, int R, int S, int[] stride, int[] padding, int[] dilation) -> Tensor");
}
TORCH_LIBRARY_IMPL(sjb200, CUDA, m) {
    m.impl("conv2d_nhwc_forward", &sjb200::conv2d_nhwc_forward);
    m.impl("conv2d_nhwc_dgrad", &sjb200::conv2d_nhwc_dgrad);
    m.impl("conv2d_nhwc_wgrad", &sjb200::conv2d_nhwc_wgrad);
}
