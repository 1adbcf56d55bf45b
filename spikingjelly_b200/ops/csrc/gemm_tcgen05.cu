// Persistent, warp-specialised 16-bit GEMM on the 5th-generation tensor cores.
//
//   D[M, N] = sum_k A[m, k] * B[n, k]          (fp32 accumulation in TMEM)
//
// * one CTA per SM, static round-robin over 128 x BN output tiles (n fastest, so the
//   CTAs that run together share the same rows of A through L2);
// * warp 0: TMA producer (one thread) filling a STAGES-deep ring of 128B-swizzled
//   A/B tiles; warp 1: tcgen05.mma issuer (one thread), accumulator double-buffered in
//   TMEM (2 x BN columns) so the epilogue of tile i overlaps the main loop of tile
//   i+1; warps 2-9: epilogue (tcgen05.ld -> convert -> shared -> TMA store), two warps per TMEM lane quarter,
//   each draining half of the tile's columns;
// * either operand may be stored "MN-major" (memory is [K, M] or [K, N] with the
//   non-contracted index contiguous), which is what dgrad/wgrad of a linear layer
//   need, so no transposes are ever materialised;
// * split-K for skinny outputs (wgrad): partial sums go to an fp32 scratch
//   [splits, M, N]; `splitk_reduce_kernel` adds them in a fixed order;
// * all mbarrier waits are bounded; on expiry the kernel records where it gave
//   up in a KernelStatus word, lets in-flight copies land, frees TMEM and returns.
#include "gemm_tcgen05_kernel.cuh"

namespace sjb200 {
using namespace tc;

// D = A (.) B with fp32 accumulation.
//   a_mn == false: `a` is [M, K] (K contiguous);  a_mn == true: `a` is [K, M] (M contiguous)
//   b_mn == false: `b` is [N, K] (K contiguous);  b_mn == true: `b` is [K, N] (N contiguous)
//   out_f32: result dtype fp32 instead of the input dtype;  split_k: 0 = choose, else forced
static at::Tensor gemm_16bit_impl(const at::Tensor& a, const at::Tensor& b, bool a_mn, bool b_mn, bool out_f32, int64_t split_k,
                                  at::Tensor* stats, const at::Tensor* into = nullptr) {
    TORCH_CHECK(a.is_cuda() && b.is_cuda(), "gemm_16bit: CUDA tensors required");
    TORCH_CHECK(a.dim() == 2 && b.dim() == 2, "gemm_16bit: 2-D operands required");
    TORCH_CHECK(a.scalar_type() == b.scalar_type() && (a.scalar_type() == at::kBFloat16 || a.scalar_type() == at::kHalf),
                "gemm_16bit: both operands must be bf16 or both fp16");
    const c10::cuda::CUDAGuard guard(a.device());
    // Autograd worker threads may not have the primary context bound yet; the driver-level
    // tensor-map encoder needs one.  A null free binds it and does nothing else.
    C10_CUDA_CHECK(cudaFree(nullptr));
    at::Tensor A = a.stride(1) == 1 ? a : a.contiguous();
    at::Tensor B = b.stride(1) == 1 ? b : b.contiguous();
    const int64_t M = a_mn ? A.size(1) : A.size(0), K = a_mn ? A.size(0) : A.size(1);
    const int64_t N = b_mn ? B.size(1) : B.size(0), Kb = b_mn ? B.size(0) : B.size(1);
    TORCH_CHECK(K == Kb, "gemm_16bit: contraction sizes differ (", K, " vs ", Kb, ")");
    TORCH_CHECK(N % 8 == 0, "gemm_16bit: N must be a multiple of 8");
    const bool bf16 = a.scalar_type() == at::kBFloat16;

    const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    // Two SMs per 256 x 256 tile where the output is large enough and the contraction long enough (>= 16 k-blocks:
    // measured, shorter main loops are bound by the epilogue, where the pair's cross-CTA hand-shakes only cost);
    // else one SM per 128 x BN tile.  Mode 2 forces the pair kernel wherever the shape allows it.
    const bool use_pair = pair_mode() != 0 && M >= 2 * BM && N >= kPairBN && sms >= 2 &&
                          (pair_mode() == 2 || (K + BK - 1) / BK >= 16);
    const int BN = use_pair ? kPairBN : (N > 128 ? 256 : 128);
    const int TM = use_pair ? 2 * BM : BM;
    const int units = use_pair ? sms / 2 : sms;            // tiles that run at the same time
    const int tiles = (int)(((M + TM - 1) / TM) * ((N + BN - 1) / BN));
    const int kb_total = (int)((K + BK - 1) / BK);
    int splits = (int)split_k;
    if (splits <= 0) {
        splits = 1;
        if (tiles * 2 <= units && kb_total >= 16) splits = std::min(std::max(1, units / tiles), kb_total / 4);
    }
    if (stats != nullptr) splits = 1;                      // the statistics come from complete 16-bit tiles
    splits = std::max(1, std::min(splits, kb_total));
    int kb_per = (kb_total + splits - 1) / splits;
    splits = (kb_total + kb_per - 1) / kb_per;

    GemmArgs g{};
    g.M = (int)M; g.N = (int)N; g.K = (int)K; g.ldd = (int)N;
    g.split_k = splits; g.kb_per_split = kb_per;
    g.out_f32 = (out_f32 || splits > 1) ? 1 : 0;
    g.ab_format = bf16 ? 1 : 0;
    g.out_bf16 = bf16 ? 1 : 0;
    g.alpha = nullptr;
    g.stats = nullptr;
    if (stats != nullptr) {
        TORCH_CHECK(!out_f32, "gemm_16bit: column statistics need a 16-bit result");
        // the pair kernel works on 256-row tiles: its last tile may cover one more (all-zero) 128-row slice
        *stats = at::empty({(M + TM - 1) / TM * (TM / BM) * 4, 2, N}, a.options().dtype(at::kFloat));
        g.stats = stats->data_ptr<float>();
    }

    const CUtensorMap ta = a_mn ? make_map(A.data_ptr(), K, M, A.stride(0), BK, bf16)
                                : make_map(A.data_ptr(), M, K, A.stride(0), BM, bf16);
    const CUtensorMap tb = b_mn ? make_map(B.data_ptr(), K, N, B.stride(0), BK, bf16)
                                : make_map(B.data_ptr(), N, K, B.stride(0), use_pair ? kPairBN / 2 : BN, bf16);

    auto opts = a.options();
    at::Tensor out;
    if (into != nullptr) {
        // the caller's buffer (e.g. one in symmetric memory that peers will read): same shape, dtype and device, contiguous
        TORCH_CHECK(into->is_cuda() && into->device() == a.device() && into->is_contiguous() && into->numel() == M * N &&
                    into->scalar_type() == (out_f32 ? at::kFloat : a.scalar_type()) &&
                    reinterpret_cast<uintptr_t>(into->data_ptr()) % 16 == 0, "gemm_16bit_into: output buffer does not fit the product");
        out = into->view({M, N});
    } else {
        out = at::empty({M, N}, out_f32 ? opts.dtype(at::kFloat) : opts);
    }
    at::Tensor scratch;
    void* dptr = out.data_ptr();
    if (splits > 1) {
        scratch = at::empty({splits, M, N}, opts.dtype(at::kFloat));
        dptr = scratch.data_ptr();
    }
    // 16-bit results leave through TMA (one 32 x 32 box per epilogue warp, 64-byte swizzle); fp32 results are stored directly
    const CUtensorMap td = g.out_f32 ? ta : make_map(out.data_ptr(), M, N, N, 32, bf16, 32);
    at::Tensor& st = status_word(a.device());
    KernelStatus* stp = reinterpret_cast<KernelStatus*>(st.data_ptr<int>());
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();

    if (use_pair) {
        const int grid = 2 * std::min(tiles * splits, units);
        if (a_mn && b_mn) launch_pair<true, true>(ta, tb, td, dptr, g, stp, grid, stream);
        else if (a_mn) launch_pair<true, false>(ta, tb, td, dptr, g, stp, grid, stream);
        else if (b_mn) launch_pair<false, true>(ta, tb, td, dptr, g, stp, grid, stream);
        else launch_pair<false, false>(ta, tb, td, dptr, g, stp, grid, stream);
    } else {
        const int grid = std::min(tiles * splits, sms);
#define SJ_LAUNCH(BN_, ST_)                                                                          \
    do {                                                                                             \
        if (a_mn && b_mn) launch<BN_, ST_, true, true>(ta, tb, td, dptr, g, stp, grid, stream);          \
        else if (a_mn) launch<BN_, ST_, true, false>(ta, tb, td, dptr, g, stp, grid, stream);            \
        else if (b_mn) launch<BN_, ST_, false, true>(ta, tb, td, dptr, g, stp, grid, stream);            \
        else launch<BN_, ST_, false, false>(ta, tb, td, dptr, g, stp, grid, stream);                     \
    } while (0)
        if (BN == 256) SJ_LAUNCH(256, 4); else SJ_LAUNCH(128, 6);
#undef SJ_LAUNCH
    }
    C10_CUDA_KERNEL_LAUNCH_CHECK();

    if (splits > 1) {
        const long long mn = (long long)M * N;
        const int threads = 256;
        const unsigned blocks = (unsigned)((mn / 4 + threads) / threads);
        if (out_f32) splitk_reduce_kernel<float><<<blocks, threads, 0, stream>>>(scratch.data_ptr<float>(), out.data_ptr<float>(), mn, splits, 0.f, nullptr);
        else if (bf16) splitk_reduce_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(scratch.data_ptr<float>(), reinterpret_cast<__nv_bfloat16*>(out.data_ptr()), mn, splits, 0.f, nullptr);
        else splitk_reduce_kernel<__half><<<blocks, threads, 0, stream>>>(scratch.data_ptr<float>(), reinterpret_cast<__half*>(out.data_ptr()), mn, splits, 0.f, nullptr);
        C10_CUDA_KERNEL_LAUNCH_CHECK();
    }
    return out;
}

at::Tensor gemm_16bit(const at::Tensor& a, const at::Tensor& b, bool a_mn, bool b_mn, bool out_f32, int64_t split_k) {
    return gemm_16bit_impl(a, b, a_mn, b_mn, out_f32, split_k, nullptr);
}

// The same product written into `out` (shape [M, N], the operands' dtype or fp32): lets a caller place the result in a
// buffer of its choosing, e.g. symmetric memory that other ranks read afterwards.
at::Tensor gemm_16bit_into(const at::Tensor& a, const at::Tensor& b, bool a_mn, bool b_mn, at::Tensor out) {
    return gemm_16bit_impl(a, b, a_mn, b_mn, out.scalar_type() == at::kFloat, 0, nullptr, &out);
}

// The same product plus partial[blk][0 | 1][n] = sum | sum of squares of D[32 * blk .. 32 * blk + 31][n] (rows past M
// count as zero), taken from the rounded 16-bit values inside the epilogue: a following batch norm needs no pass over D.
std::tuple<at::Tensor, at::Tensor> gemm_16bit_stats(const at::Tensor& a, const at::Tensor& b, bool a_mn, bool b_mn) {
    at::Tensor stats;
    at::Tensor out = gemm_16bit_impl(a, b, a_mn, b_mn, false, 1, &stats);
    return {out, stats};
}

// D[M, N] (bf16) = alpha * alpha2 * A[M, K] (.) B[N, K]^T with fp8 operands (each e4m3 or e5m2, K contiguous) and fp32
// accumulation on the tensor cores.  `alpha`, `alpha2`: optional fp32 device scalars (the two de-quantisation
// scales), multiplied in the epilogue so that neither a host synchronisation nor a scalar-product kernel is needed.
at::Tensor gemm_fp8(const at::Tensor& a, const at::Tensor& b, const c10::optional<at::Tensor>& alpha, bool out_f32,
                    int64_t split_k, const c10::optional<at::Tensor>& alpha2, const c10::optional<at::Tensor>& bias) {
    TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.dim() == 2 && b.dim() == 2, "gemm_fp8: 2-D CUDA operands required");
    auto fmt = [](const at::Tensor& t) { return t.scalar_type() == at::kFloat8_e4m3fn ? 0 : t.scalar_type() == at::kFloat8_e5m2 ? 1 : -1; };
    const int fa = fmt(a), fb = fmt(b);
    TORCH_CHECK(fa >= 0 && fb >= 0, "gemm_fp8: operands must be float8_e4m3fn or float8_e5m2");
    const c10::cuda::CUDAGuard guard(a.device());
    C10_CUDA_CHECK(cudaFree(nullptr));
    at::Tensor A = a.stride(1) == 1 ? a : a.contiguous();
    at::Tensor B = b.stride(1) == 1 ? b : b.contiguous();
    const int64_t M = A.size(0), K = A.size(1), N = B.size(0);
    TORCH_CHECK(B.size(1) == K, "gemm_fp8: contraction sizes differ (", K, " vs ", B.size(1), ")");
    TORCH_CHECK(N % 8 == 0 && K % 16 == 0, "gemm_fp8: N must be a multiple of 8 and K a multiple of 16");
    constexpr int BKE = 128;
    const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    const bool use_pair = pair_mode() != 0 && M >= 2 * BM && N >= kPairBN && sms >= 2 &&
                          (pair_mode() == 2 || (K + BKE - 1) / BKE >= 16);
    const int BN = use_pair ? kPairBN : (N > 128 ? 256 : 128);
    const int TM = use_pair ? 2 * BM : BM;
    const int units = use_pair ? sms / 2 : sms;
    const int tiles = (int)(((M + TM - 1) / TM) * ((N + BN - 1) / BN));
    const int kb_total = (int)((K + BKE - 1) / BKE);
    int splits = (int)split_k;
    if (splits <= 0) {
        splits = 1;
        if (tiles * 2 <= units && kb_total >= 16) splits = std::min(std::max(1, units / tiles), kb_total / 4);
    }
    splits = std::max(1, std::min(splits, kb_total));
    const int kb_per = (kb_total + splits - 1) / splits;
    splits = (kb_total + kb_per - 1) / kb_per;

    GemmArgs g{};
    g.M = (int)M; g.N = (int)N; g.K = (int)K; g.ldd = (int)N;
    g.split_k = splits; g.kb_per_split = kb_per;
    g.out_f32 = (out_f32 || splits > 1) ? 1 : 0;
    g.ab_format = fa | (fb << 4) | 0x80;
    g.out_bf16 = 1;
    g.alpha = nullptr;
    g.alpha2 = nullptr;
    g.bias = nullptr;
    at::Tensor bias_f32;
    if (bias.has_value() && bias->defined()) {
        TORCH_CHECK(bias->is_cuda() && bias->numel() == N, "gemm_fp8: bias must hold one value per output column");
        bias_f32 = bias->to(at::kFloat).contiguous();
        g.bias = bias_f32.data_ptr<float>();
    }
    if (alpha2.has_value() && alpha2->defined()) {
        TORCH_CHECK(alpha.has_value() && alpha->defined(), "gemm_fp8: alpha2 needs alpha");
        TORCH_CHECK(alpha2->is_cuda() && alpha2->scalar_type() == at::kFloat && alpha2->numel() == 1, "gemm_fp8: alpha2 must be one fp32 value on the device");
        g.alpha2 = alpha2->data_ptr<float>();
    }
    if (alpha.has_value() && alpha->defined()) {
        TORCH_CHECK(alpha->is_cuda() && alpha->scalar_type() == at::kFloat && alpha->numel() == 1, "gemm_fp8: alpha must be one fp32 value on the device");
        g.alpha = alpha->data_ptr<float>();
    }
    const CUtensorMap ta = make_map_u8(A.data_ptr(), M, K, A.stride(0), BM);
    const CUtensorMap tb = make_map_u8(B.data_ptr(), N, K, B.stride(0), use_pair ? kPairBN / 2 : BN);
    auto opts = a.options();
    at::Tensor out = at::empty({M, N}, opts.dtype(out_f32 ? at::kFloat : at::kBFloat16));
    at::Tensor scratch;
    void* dptr = out.data_ptr();
    if (splits > 1) {
        scratch = at::empty({splits, M, N}, opts.dtype(at::kFloat));
        dptr = scratch.data_ptr();
    }
    const CUtensorMap td = g.out_f32 ? ta : make_map(out.data_ptr(), M, N, N, 32, true, 32);
    at::Tensor& st = status_word(a.device());
    KernelStatus* stp = reinterpret_cast<KernelStatus*>(st.data_ptr<int>());
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    if (use_pair) launch_pair<false, false, 1>(ta, tb, td, dptr, g, stp, 2 * std::min(tiles * splits, units), stream);
    else if (BN == 256) launch<256, 4, false, false, 1>(ta, tb, td, dptr, g, stp, std::min(tiles * splits, sms), stream);
    else launch<128, 6, false, false, 1>(ta, tb, td, dptr, g, stp, std::min(tiles * splits, sms), stream);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    if (splits > 1) {
        const long long mn = (long long)M * N;
        const unsigned blocks = (unsigned)((mn / 4 + 256) / 256);
        if (out_f32) splitk_reduce_kernel<float><<<blocks, 256, 0, stream>>>(scratch.data_ptr<float>(), out.data_ptr<float>(), mn, splits, 0.f, nullptr);
        else splitk_reduce_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(scratch.data_ptr<float>(), reinterpret_cast<__nv_bfloat16*>(out.data_ptr()), mn, splits, 0.f, nullptr);
        C10_CUDA_KERNEL_LAUNCH_CHECK();
    }
    return out;
}

// Switches the CTA-pair kernel on (1) or off (0) for the shapes it supports; returns the previous setting.
int64_t gemm_set_pair_mode(int64_t mode) {
    const int prev = pair_mode();
    pair_mode() = (int)mode;
    return prev;
}

// (code, block, detail) of the first bounded wait that gave up since the last call; resets it.
std::vector<int64_t> gemm_status(const at::Tensor& like) {
    at::Tensor& st = status_word(like.device());
    at::Tensor h = st.cpu();
    st.zero_();
    auto acc = h.accessor<int, 1>();
    return {acc[0], acc[1], acc[2]};
}

}  // namespace sjb200

TORCH_LIBRARY_FRAGMENT(sjb200, m) {
    m.def("gemm_16bit(Tensor a, Tensor b, bool a_mn, bool b_mn, bool out_f32, int split_k) -> Tensor");
    m.def("gemm_16bit_stats(Tensor a, Tensor b, bool a_mn, bool b_mn) -> (Tensor, Tensor)");
    m.def("gemm_16bit_into(Tensor a, Tensor b, bool a_mn, bool b_mn, Tensor(a!) out) -> Tensor(a!)");
    m.def("gemm_fp8(Tensor a, Tensor b, Tensor? alpha, bool out_f32, int split_k, Tensor? alpha2=None, Tensor? bias=None) -> Tensor");
    m.def("gemm_status(Tensor like) -> int[]");
    m.def("gemm_set_pair_mode(int mode) -> int");
}
TORCH_LIBRARY_IMPL(sjb200, CompositeExplicitAutograd, m) {
    m.impl("gemm_set_pair_mode", &sjb200::gemm_set_pair_mode);
}
TORCH_LIBRARY_IMPL(sjb200, CUDA, m) {
    m.impl("gemm_16bit", &sjb200::gemm_16bit);
    m.impl("gemm_16bit_stats", &sjb200::gemm_16bit_stats);
    m.impl("gemm_16bit_into", &sjb200::gemm_16bit_into);
    m.impl("gemm_fp8", &sjb200::gemm_fp8);
    m.impl("gemm_status", &sjb200::gemm_status);
}
