// Spiking self-attention core:  O = scale * Q (K^T V)  per (time step, sample, head), no softmax.
//
// Inputs are the spike tensors of one fused QKV projection, channels-last:
//   S [T, B, L, 3, H, D]  (q, k, v stacked along the channel axis);  O [T, B, L, H, D].
// One CTA owns one (t, b, head): it stages Q, K, V (and dO in backward) in shared memory, forms
// the D x D matrix K^T V once and applies it to all L tokens — O(L D^2) work instead of the
// O(L^2 D) of softmax attention, and nothing of size L x L ever exists.
//   backward:  dKV = scale Q^T dO;  dQ = scale dO (K^T V)^T;  dK = V dKV^T;  dV = K dKV.
// fp32 accumulation; operands may be any 16-bit floats (spikes after a residual add need not be
// binary), so the arithmetic is exact for spike inputs whenever L < 2^24.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "common.cuh"

namespace sjb200 {
namespace {

constexpr int kThreads = 256;

template <typename T, int D>
__device__ __forceinline__ void stage_rows(const T* __restrict__ g, long long row_stride, int L, T* __restrict__ s) {
    constexpr int CH = D / 8;   // 16-byte chunks per row
    for (int i = threadIdx.x; i < L * CH; i += blockDim.x) {
        const int l = i / CH, c = i % CH;
        *reinterpret_cast<int4*>(s + l * D + c * 8) = *reinterpret_cast<const int4*>(g + (long long)l * row_stride + c * 8);
    }
}

// out[i][j] = alpha * sum_l A[l][i] * Bm[l][j]   (A, Bm: [L][D] in smem; out: [D][D+1] fp32 in smem)
template <typename T, int D>
__device__ __forceinline__ void outer_accumulate(const T* __restrict__ A, const T* __restrict__ Bm, int L, float alpha,
                                                 float* __restrict__ out) {
    constexpr int TD = D / 4;
    for (int tile = threadIdx.x; tile < TD * TD; tile += blockDim.x) {
        const int i0 = (tile / TD) * 4, j0 = (tile % TD) * 4;
        float acc[4][4] = {};
        for (int l = 0; l < L; ++l) {
            float a[4], b[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) { a[q] = to_f32<T>(A[l * D + i0 + q]); b[q] = to_f32<T>(Bm[l * D + j0 + q]); }
#pragma unroll
            for (int p = 0; p < 4; ++p)
#pragma unroll
                for (int q = 0; q < 4; ++q) acc[p][q] = fmaf(a[p], b[q], acc[p][q]);
        }
#pragma unroll
        for (int p = 0; p < 4; ++p)
#pragma unroll
            for (int q = 0; q < 4; ++q) out[(i0 + p) * (D + 1) + j0 + q] = alpha * acc[p][q];
    }
}

// dst[l][j] = alpha * sum_i A[l][i] * M[i][j]  (TRANS = false)   or   alpha * sum_i A[l][i] * M[j][i]  (TRANS = true)
// A: [L][D] smem; M: [D][D+1] fp32 smem; dst: global, row stride `dst_stride`
template <typename T, int D, bool TRANS>
__device__ __forceinline__ void apply_matrix(const T* __restrict__ A, const float* __restrict__ M, int L, float alpha,
                                             T* __restrict__ dst, long long dst_stride) {
    constexpr int TD = D / 4;
    const int row_tiles = (L + 3) / 4;
    for (int tile = threadIdx.x; tile < row_tiles * TD; tile += blockDim.x) {
        const int l0 = (tile / TD) * 4, j0 = (tile % TD) * 4;
        float acc[4][4] = {};
        for (int i = 0; i < D; ++i) {
            float a[4], m[4];
#pragma unroll
            for (int p = 0; p < 4; ++p) a[p] = (l0 + p < L) ? to_f32<T>(A[(l0 + p) * D + i]) : 0.0f;
#pragma unroll
            for (int q = 0; q < 4; ++q) m[q] = TRANS ? M[(j0 + q) * (D + 1) + i] : M[i * (D + 1) + j0 + q];
#pragma unroll
            for (int p = 0; p < 4; ++p)
#pragma unroll
                for (int q = 0; q < 4; ++q) acc[p][q] = fmaf(a[p], m[q], acc[p][q]);
        }
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            if (l0 + p < L) {
                Pack<T, 4> o;
#pragma unroll
                for (int q = 0; q < 4; ++q) o.e[q] = from_f32<T>(alpha * acc[p][q]);
                *reinterpret_cast<Pack<T, 4>*>(dst + (long long)(l0 + p) * dst_stride + j0) = o;
            }
        }
    }
}

template <typename T, int D>
__global__ void __launch_bounds__(kThreads)
ssa_forward_kernel(const T* __restrict__ S, T* __restrict__ O, int L, int H, float scale) {
    extern __shared__ __align__(16) uint8_t smem[];
    T* Qs = reinterpret_cast<T*>(smem);
    T* Ks = Qs + L * D;
    T* Vs = Ks + L * D;
    float* KV = reinterpret_cast<float*>(Vs + L * D);
    const int C = H * D;
    const int head = blockIdx.x % H;
    const long long tb = blockIdx.x / H;
    const T* base = S + tb * L * 3 * C + head * D;
    stage_rows<T, D>(base, 3LL * C, L, Qs);
    stage_rows<T, D>(base + C, 3LL * C, L, Ks);
    stage_rows<T, D>(base + 2 * C, 3LL * C, L, Vs);
    __syncthreads();
    outer_accumulate<T, D>(Ks, Vs, L, 1.0f, KV);
    __syncthreads();
    apply_matrix<T, D, false>(Qs, KV, L, scale, O + tb * L * C + head * D, C);
}

template <typename T, int D>
__global__ void __launch_bounds__(kThreads)
ssa_backward_kernel(const T* __restrict__ S, const T* __restrict__ dO, T* __restrict__ dS, int L, int H, float scale) {
    extern __shared__ __align__(16) uint8_t smem[];
    T* Qs = reinterpret_cast<T*>(smem);
    T* Ks = Qs + L * D;
    T* Vs = Ks + L * D;
    T* Gs = Vs + L * D;
    float* KV = reinterpret_cast<float*>(Gs + L * D);
    float* dKV = KV + D * (D + 1);
    const int C = H * D;
    const int head = blockIdx.x % H;
    const long long tb = blockIdx.x / H;
    const T* base = S + tb * L * 3 * C + head * D;
    stage_rows<T, D>(base, 3LL * C, L, Qs);
    stage_rows<T, D>(base + C, 3LL * C, L, Ks);
    stage_rows<T, D>(base + 2 * C, 3LL * C, L, Vs);
    stage_rows<T, D>(dO + tb * L * C + head * D, C, L, Gs);
    __syncthreads();
    outer_accumulate<T, D>(Ks, Vs, L, 1.0f, KV);        // K^T V
    outer_accumulate<T, D>(Qs, Gs, L, scale, dKV);      // scale Q^T dO
    __syncthreads();
    T* dbase = dS + tb * L * 3 * C + head * D;
    apply_matrix<T, D, true>(Gs, KV, L, scale, dbase, 3LL * C);          // dQ = scale dO KV^T
    apply_matrix<T, D, true>(Vs, dKV, L, 1.0f, dbase + C, 3LL * C);      // dK = V dKV^T
    apply_matrix<T, D, false>(Ks, dKV, L, 1.0f, dbase + 2 * C, 3LL * C); // dV = K dKV
}

size_t smem_bytes(int L, int D, int n_mats, int n_sq) { return (size_t)n_mats * L * D * 2 + (size_t)n_sq * D * (D + 1) * 4; }

template <typename T, int D>
void launch_fwd(const at::Tensor& S, at::Tensor& O, int TB, int L, int H, float scale, cudaStream_t st) {
    const size_t sm = smem_bytes(L, D, 3, 1);
    auto k = ssa_forward_kernel<T, D>;
    C10_CUDA_CHECK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm));
    k<<<TB * H, kThreads, sm, st>>>(reinterpret_cast<const T*>(S.data_ptr()), reinterpret_cast<T*>(O.data_ptr()), L, H, scale);
}
template <typename T, int D>
void launch_bwd(const at::Tensor& S, const at::Tensor& dO, at::Tensor& dS, int TB, int L, int H, float scale, cudaStream_t st) {
    const size_t sm = smem_bytes(L, D, 4, 2);
    auto k = ssa_backward_kernel<T, D>;
    C10_CUDA_CHECK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm));
    k<<<TB * H, kThreads, sm, st>>>(reinterpret_cast<const T*>(S.data_ptr()), reinterpret_cast<const T*>(dO.data_ptr()),
                                    reinterpret_cast<T*>(dS.data_ptr()), L, H, scale);
}

void check(const at::Tensor& S, int64_t L, int64_t H) {
    TORCH_CHECK(S.is_cuda() && S.is_contiguous(), "ssa: contiguous CUDA tensor required");
    TORCH_CHECK(S.scalar_type() == at::kBFloat16 || S.scalar_type() == at::kHalf, "ssa: bf16 or fp16 required");
    const int64_t C3 = S.size(-1);
    TORCH_CHECK(C3 % (3 * H) == 0, "ssa: last dimension must be 3 * heads * head_dim");
    const int64_t D = C3 / (3 * H);
    TORCH_CHECK(D == 32 || D == 64, "ssa: head_dim must be 32 or 64");
    TORCH_CHECK(S.numel() % (L * C3) == 0, "ssa: tokens per sample do not divide the tensor");
    TORCH_CHECK(smem_bytes((int)L, (int)D, 4, 2) <= 220 * 1024, "ssa: sequence too long for the shared-memory kernel");
}

}  // namespace

// S: [..., L, 3*H*D] -> O: [..., L, H*D]
at::Tensor ssa_forward(const at::Tensor& S, int64_t L, int64_t H, double scale) {
    check(S, L, H);
    const c10::cuda::CUDAGuard guard(S.device());
    const int64_t C = S.size(-1) / 3, D = C / H;
    std::vector<int64_t> shape(S.sizes().begin(), S.sizes().end());
    shape.back() = C;
    at::Tensor O = at::empty(shape, S.options());
    const int TB = (int)(S.numel() / (L * 3 * C));
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    const bool bf = S.scalar_type() == at::kBFloat16;
    if (D == 64) { if (bf) launch_fwd<__nv_bfloat16, 64>(S, O, TB, (int)L, (int)H, (float)scale, st); else launch_fwd<__half, 64>(S, O, TB, (int)L, (int)H, (float)scale, st); }
    else { if (bf) launch_fwd<__nv_bfloat16, 32>(S, O, TB, (int)L, (int)H, (float)scale, st); else launch_fwd<__half, 32>(S, O, TB, (int)L, (int)H, (float)scale, st); }
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return O;
}

at::Tensor ssa_backward(const at::Tensor& dO, const at::Tensor& S, int64_t L, int64_t H, double scale) {
    check(S, L, H);
    const c10::cuda::CUDAGuard guard(S.device());
    const int64_t C = S.size(-1) / 3, D = C / H;
    at::Tensor g = dO.to(S.scalar_type()).contiguous();
    at::Tensor dS = at::empty_like(S);
    const int TB = (int)(S.numel() / (L * 3 * C));
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    const bool bf = S.scalar_type() == at::kBFloat16;
    if (D == 64) { if (bf) launch_bwd<__nv_bfloat16, 64>(S, g, dS, TB, (int)L, (int)H, (float)scale, st); else launch_bwd<__half, 64>(S, g, dS, TB, (int)L, (int)H, (float)scale, st); }
    else { if (bf) launch_bwd<__nv_bfloat16, 32>(S, g, dS, TB, (int)L, (int)H, (float)scale, st); else launch_bwd<__half, 32>(S, g, dS, TB, (int)L, (int)H, (float)scale, st); }
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return dS;
}

}  // namespace sjb200

TORCH_LIBRARY_FRAGMENT(sjb200, m) {
    m.def("ssa_forward(Tensor S, int L, int H, float scale) -> Tensor");
    m.def("ssa_backward(Tensor dO, Tensor S, int L, int H, float scale) -> Tensor");
}
TORCH_LIBRARY_IMPL(sjb200, CUDA, m) {
    m.impl("ssa_forward", &sjb200::ssa_forward);
    m.impl("ssa_backward", &sjb200::ssa_backward);
}
