// Spiking self-attention core:  O = scale * Q (K^T V)  per (time step, sample, head), no softmax.
//
// Inputs are the spike tensors of one fused QKV projection, channels-last:
//   S [T, B, L, 3, H, D]  (q, k, v stacked along the channel axis);  O [T, B, L, H, D].
// One CTA owns one (t, b, head): it stages Q, K, V (and dO in backward) in shared memory, forms
// the D x D matrix K^T V once and applies it to all L tokens — O(L D^2) work instead of the
// O(L^2 D) of softmax attention, and nothing of size L x L ever exists.
//   backward:  dKV = scale Q^T dO;  dQ = scale dO (K^T V)^T;  dK = V dKV^T;  dV = K dKV.
//
// All six products are warp-level m16n8k16 tensor-core MMAs (16-bit operands, fp32 accumulation)
// fed by ldmatrix from padded shared-memory tiles; the per-head problems (64 x 64 x L and
// L x 64 x 64) are far below one tcgen05 tile, so the CTA-wide UMMA path would idle most of its
// 128 x 256 datapath here.  K^T V of binary spikes is an integer <= L and therefore exact in bf16 for
// L <= 256; dKV is rounded to the operand dtype once, like the batched-matmul formulation it replaces.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "common.cuh"

namespace sjb200 {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

template <int D> struct Geo {
    static constexpr int LD = D + 8;          // padded row length (elements): 16-byte rows shifted by 4 banks
};

// ---- fragment helpers -----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t s_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <typename T> __device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <> __device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <> __device__ __forceinline__ void mma16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi); return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi); return *reinterpret_cast<uint32_t*>(&v);
}

// Stage `rows` rows of D contiguous elements (row stride `gstride` in global) into a padded tile with
// asynchronous 16-byte copies (no register round trip: every copy of the tile is in flight at once, which is
// what hides the DRAM latency with a single resident CTA per SM) and zero rows [rows, rows_pad).
// The caller commits the group and waits for it.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }

template <typename T, int D>
__device__ __forceinline__ void stage(const T* __restrict__ g, long long gstride, int rows, int rows_pad, T* __restrict__ s) {
    constexpr int CH = D / 8, LD = Geo<D>::LD;
    for (int i = threadIdx.x; i < rows_pad * CH; i += blockDim.x) {
        const int l = i / CH, c = i % CH;
        if (l < rows) cp_async16(s_addr(s + l * LD + c * 8), g + (long long)l * gstride + c * 8);
        else *reinterpret_cast<int4*>(s + l * LD + c * 8) = make_int4(0, 0, 0, 0);
    }
}

// out[i][j] = alpha * sum_l X[l][i] * Y[l][j]  for i, j in [0, D);  X, Y: padded tiles with Lp rows (Lp % 16 == 0).
// Result rounded to T and stored in the padded tile `out` ([D][LD]).
template <typename T, int D>
__device__ __forceinline__ void gram(const T* __restrict__ X, const T* __restrict__ Y, int Lp, float alpha, T* __restrict__ out) {
    constexpr int LD = Geo<D>::LD;
    constexpr int MT = D / 16, NT = D / 8;               // m16 / n8 tiles of the D x D result
    constexpr int NT_W = (MT * NT) / kWarps;             // n8 tiles per warp (4 for D = 64, 1 for D = 32)
    static_assert((MT * NT) % kWarps == 0 && NT_W >= 1, "tile split");
    constexpr int W_PER_M = NT / NT_W;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = (warp / W_PER_M) * 16, n0 = (warp % W_PER_M) * NT_W * 8;
    float acc[NT_W][4] = {};
    const int sub = lane >> 3, r = lane & 7;             // ldmatrix: lane supplies row r of 8x8 matrix `sub`
    for (int k0 = 0; k0 < Lp; k0 += 16) {
        // A fragment of X^T: stored block (k-half, m-half) -> a0:(k0,m0) a1:(k0,m0+8) a2:(k0+8,m0) a3:(k0+8,m0+8)
        uint32_t a[4];
        ldsm_x4_t(s_addr(X + (k0 + (sub >> 1) * 8 + r) * LD + m0 + (sub & 1) * 8), a);
#pragma unroll
        for (int nt = 0; nt < NT_W; nt += 2) {
            // B fragments of Y (stored [k][n]): matrices (k0,n) (k0+8,n) (k0,n+8) (k0+8,n+8)
            uint32_t b[4];
            ldsm_x4_t(s_addr(Y + (k0 + (sub & 1) * 8 + r) * LD + n0 + nt * 8 + (sub >> 1) * 8), b);
            mma16816<T>(acc[nt], a, b[0], b[1]);
            if (nt + 1 < NT_W) mma16816<T>(acc[nt + 1 < NT_W ? nt + 1 : nt], a, b[2], b[3]);
        }
    }
    const int row = m0 + (lane >> 2), col = (lane & 3) * 2;
#pragma unroll
    for (int nt = 0; nt < NT_W; ++nt) {
        *reinterpret_cast<uint32_t*>(out + row * LD + n0 + nt * 8 + col) = pack2<T>(alpha * acc[nt][0], alpha * acc[nt][1]);
        *reinterpret_cast<uint32_t*>(out + (row + 8) * LD + n0 + nt * 8 + col) = pack2<T>(alpha * acc[nt][2], alpha * acc[nt][3]);
    }
}

// dst[l][j] = alpha * sum_c X[l][c] * M[c][j]  (TRANS = false)   or   alpha * sum_c X[l][c] * M[j][c]  (TRANS = true)
// X: padded tile (Lp rows; overwritten with the result), M: padded [D][LD] tile; dst: global, row stride `dstride`, rows l < L.
template <typename T, int D, bool TRANS>
__device__ __forceinline__ void apply(T* __restrict__ X, const T* __restrict__ M, int L, int Lp, float alpha,
                                      T* __restrict__ dst, long long dstride) {
    constexpr int LD = Geo<D>::LD, NT = D / 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane >> 3, r = lane & 7;
    for (int m0 = warp * 16; m0 < Lp; m0 += kWarps * 16) {
        float acc[NT][4] = {};
#pragma unroll
        for (int k0 = 0; k0 < D; k0 += 16) {
            uint32_t a[4];   // a0:(m0,k0) a1:(m0+8,k0) a2:(m0,k0+8) a3:(m0+8,k0+8)
            ldsm_x4(s_addr(X + (m0 + (sub & 1) * 8 + r) * LD + k0 + (sub >> 1) * 8), a);
#pragma unroll
            for (int nt = 0; nt < NT; nt += 2) {
                uint32_t b[4];   // b0,b1: n-tile nt (k0, k0+8);  b2,b3: n-tile nt+1
                if (TRANS) ldsm_x4(s_addr(M + (nt * 8 + (sub >> 1) * 8 + r) * LD + k0 + (sub & 1) * 8), b);
                else ldsm_x4_t(s_addr(M + (k0 + (sub & 1) * 8 + r) * LD + nt * 8 + (sub >> 1) * 8), b);
                mma16816<T>(acc[nt], a, b[0], b[1]);
                mma16816<T>(acc[nt + 1], a, b[2], b[3]);
            }
        }
        // Rows [m0, m0 + 16) of X are read by this warp only and are dead now: the result goes back into them, and
        // leaves as 16-byte stores of whole 2 * D-byte rows instead of 4-byte fragments.
        __syncwarp();
        const int row = m0 + (lane >> 2), col = (lane & 3) * 2;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            *reinterpret_cast<uint32_t*>(X + row * LD + nt * 8 + col) = pack2<T>(alpha * acc[nt][0], alpha * acc[nt][1]);
            *reinterpret_cast<uint32_t*>(X + (row + 8) * LD + nt * 8 + col) = pack2<T>(alpha * acc[nt][2], alpha * acc[nt][3]);
        }
        __syncwarp();
        constexpr int CH = D / 8;
#pragma unroll
        for (int i = lane; i < 16 * CH; i += 32) {
            const int l = m0 + i / CH, c = i % CH;
            if (l < L) *reinterpret_cast<int4*>(dst + (long long)l * dstride + c * 8) = *reinterpret_cast<const int4*>(X + l * LD + c * 8);
        }
    }
}

template <typename T, int D>
__global__ void __launch_bounds__(kThreads)
ssa_forward_kernel(const T* __restrict__ S, T* __restrict__ O, int L, int Lp, int H, float scale) {
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int LD = Geo<D>::LD;
    T* Qs = reinterpret_cast<T*>(smem);
    T* Ks = Qs + Lp * LD;
    T* Vs = Ks + Lp * LD;
    T* KV = Vs + Lp * LD;            // [D][LD]
    const int C = H * D;
    const int head = blockIdx.x % H;
    const long long tb = blockIdx.x / H;
    const T* base = S + tb * L * 3 * C + head * D;
    stage<T, D>(base + C, 3LL * C, L, Lp, Ks);
    stage<T, D>(base + 2 * C, 3LL * C, L, Lp, Vs);
    cp_async_commit();
    stage<T, D>(base, 3LL * C, L, Lp, Qs);
    cp_async_commit();
    cp_async_wait<1>();                       // K and V have landed; Q is still in flight under the gram
    __syncthreads();
    gram<T, D>(Ks, Vs, Lp, 1.0f, KV);
    cp_async_wait<0>();
    __syncthreads();
    apply<T, D, false>(Qs, KV, L, Lp, scale, O + tb * L * C + head * D, C);
}

template <typename T, int D>
__global__ void __launch_bounds__(kThreads)
ssa_backward_kernel(const T* __restrict__ S, const T* __restrict__ dO, T* __restrict__ dS, int L, int Lp, int H, float scale) {
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int LD = Geo<D>::LD;
    T* Qs = reinterpret_cast<T*>(smem);
    T* Ks = Qs + Lp * LD;
    T* Vs = Ks + Lp * LD;
    T* Gs = Vs + Lp * LD;
    T* KV = Gs + Lp * LD;
    T* dKV = KV + D * LD;
    const int C = H * D;
    const int head = blockIdx.x % H;
    const long long tb = blockIdx.x / H;
    const T* base = S + tb * L * 3 * C + head * D;
    stage<T, D>(base + C, 3LL * C, L, Lp, Ks);
    stage<T, D>(base + 2 * C, 3LL * C, L, Lp, Vs);
    cp_async_commit();
    stage<T, D>(base, 3LL * C, L, Lp, Qs);
    stage<T, D>(dO + tb * L * C + head * D, C, L, Lp, Gs);
    cp_async_commit();
    cp_async_wait<1>();                       // K and V have landed; Q and dO are still in flight under the first gram
    __syncthreads();
    gram<T, D>(Ks, Vs, Lp, 1.0f, KV);         // K^T V
    cp_async_wait<0>();
    __syncthreads();
    gram<T, D>(Qs, Gs, Lp, scale, dKV);       // scale Q^T dO
    __syncthreads();
    T* dbase = dS + tb * L * 3 * C + head * D;
    apply<T, D, true>(Gs, KV, L, Lp, scale, dbase, 3LL * C);           // dQ[l][i] = scale sum_j dO[l][j] KV[i][j]
    apply<T, D, true>(Vs, dKV, L, Lp, 1.0f, dbase + C, 3LL * C);       // dK[l][i] = sum_j V[l][j] dKV[i][j]
    apply<T, D, false>(Ks, dKV, L, Lp, 1.0f, dbase + 2 * C, 3LL * C);  // dV[l][j] = sum_i K[l][i] dKV[i][j]
}

int pad16(int64_t L) { return (int)((L + 15) / 16 * 16); }
size_t smem_bytes(int Lp, int D, int n_mats, int n_sq) { return ((size_t)n_mats * Lp + (size_t)n_sq * D) * (D + 8) * 2; }

template <typename T, int D>
void launch_fwd(const at::Tensor& S, at::Tensor& O, int TB, int L, int H, float scale, cudaStream_t st) {
    const int Lp = pad16(L);
    const size_t sm = smem_bytes(Lp, D, 3, 1);
    auto k = ssa_forward_kernel<T, D>;
    C10_CUDA_CHECK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm));
    k<<<TB * H, kThreads, sm, st>>>(reinterpret_cast<const T*>(S.data_ptr()), reinterpret_cast<T*>(O.data_ptr()), L, Lp, H, scale);
}
template <typename T, int D>
void launch_bwd(const at::Tensor& S, const at::Tensor& dO, at::Tensor& dS, int TB, int L, int H, float scale, cudaStream_t st) {
    const int Lp = pad16(L);
    const size_t sm = smem_bytes(Lp, D, 4, 2);
    auto k = ssa_backward_kernel<T, D>;
    C10_CUDA_CHECK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm));
    k<<<TB * H, kThreads, sm, st>>>(reinterpret_cast<const T*>(S.data_ptr()), reinterpret_cast<const T*>(dO.data_ptr()),
                                    reinterpret_cast<T*>(dS.data_ptr()), L, Lp, H, scale);
}

void check(const at::Tensor& S, int64_t L, int64_t H) {
    TORCH_CHECK(S.is_cuda() && S.is_contiguous(), "ssa: contiguous CUDA tensor required");
    TORCH_CHECK(S.scalar_type() == at::kBFloat16 || S.scalar_type() == at::kHalf, "ssa: bf16 or fp16 required");
    const int64_t C3 = S.size(-1);
    TORCH_CHECK(C3 % (3 * H) == 0, "ssa: last dimension must be 3 * heads * head_dim");
    const int64_t D = C3 / (3 * H);
    TORCH_CHECK(D == 32 || D == 64, "ssa: head_dim must be 32 or 64");
    TORCH_CHECK(S.numel() % (L * C3) == 0, "ssa: tokens per sample do not divide the tensor");
    TORCH_CHECK(smem_bytes(pad16(L), (int)D, 4, 2) <= 220 * 1024, "ssa: sequence too long for the shared-memory kernel");
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
