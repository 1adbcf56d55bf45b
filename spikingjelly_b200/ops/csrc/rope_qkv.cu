// Rotary position embedding fused with the split of a packed QKV projection.
//
//   qkv  [N, S, H, 3, D]   16-bit, contiguous: the output of one linear layer whose rows are ordered head-major
//                           (so that tensor parallelism shards whole heads); N = time steps x batch
//   cos, sin [>= S, D]     fp32 tables; entry [s, i] for i < D/2 is the angle of the pair (i, i + D/2) (half-split form)
//   q, k, v [N, S, H, D]   contiguous; q and k rotated, v copied.  Attention takes them as [N, H, S, D] views, and its
//                           output comes back in the same memory order, i.e. already laid out as [N, S, H * D] rows.
//
// The eager form (two concatenations, four multiplications and two additions on strided views, then copies to make
// the operands contiguous) was the largest single item of the language-model step; this is one pass: read 3 D, write 3 D.
// Backward applies the inverse rotation to the gradients of q and k and packs the three gradients back into [N, S, H, 3, D].
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "common.cuh"

namespace sjb200 {
namespace {

constexpr int V = 8;

// SIGN = +1: forward rotation;  -1: inverse (gradient).  PACK = false: packed -> three tensors;  true: three -> packed.
template <typename T, int SIGN, bool PACK>
__global__ void __launch_bounds__(256)
rope_qkv_kernel(const T* __restrict__ packed_in, T* __restrict__ packed_out, const T* __restrict__ q_in, const T* __restrict__ k_in,
                const T* __restrict__ v_in, T* __restrict__ q_out, T* __restrict__ k_out, T* __restrict__ v_out,
                const float* __restrict__ cos_t, const float* __restrict__ sin_t, long long rows, int S, int H, int D, int offset) {
    const int half = D / 2, cpr = half / V;                       // 16-byte chunks per half row
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * cpr) return;
    const long long row = idx / cpr;                                // (n, s, h)
    const int c = (int)(idx - row * cpr) * V;
    const int s = (int)((row / H) % S);
    float cs[V], sn[V];
    load_vec<float, V>(cos_t + (long long)(s + offset) * D + c, cs);
    load_vec<float, V>(sin_t + (long long)(s + offset) * D + c, sn);
    const long long po = row * 3 * D, so = row * D;                 // packed / split offsets of this (n, s, h)
#pragma unroll
    for (int which = 0; which < 3; ++which) {
        const T* src_lo = PACK ? (which == 0 ? q_in : which == 1 ? k_in : v_in) + so + c : packed_in + po + which * D + c;
        T* dst_lo = PACK ? packed_out + po + which * D + c : (which == 0 ? q_out : which == 1 ? k_out : v_out) + so + c;
        float lo[V], hi[V];
        load_vec_stream<T, V>(src_lo, lo);
        load_vec_stream<T, V>(src_lo + half, hi);
        if (which < 2) {
            float a[V], b[V];
#pragma unroll
            for (int j = 0; j < V; ++j) {
                a[j] = lo[j] * cs[j] - (float)SIGN * hi[j] * sn[j];
                b[j] = hi[j] * cs[j] + (float)SIGN * lo[j] * sn[j];
            }
            store_vec<T, V>(dst_lo, a);
            store_vec<T, V>(dst_lo + half, b);
        } else {
            store_vec<T, V>(dst_lo, lo);
            store_vec<T, V>(dst_lo + half, hi);
        }
    }
}

void check_tables(const at::Tensor& cos_t, const at::Tensor& sin_t, int64_t S, int64_t D, int64_t offset) {
    TORCH_CHECK(cos_t.is_cuda() && sin_t.is_cuda() && cos_t.scalar_type() == at::kFloat && sin_t.scalar_type() == at::kFloat &&
                cos_t.is_contiguous() && sin_t.is_contiguous() && cos_t.dim() == 2 && cos_t.sizes() == sin_t.sizes() &&
                cos_t.size(1) == D && cos_t.size(0) >= S + offset, "rope_qkv: cos / sin must be contiguous fp32 [>= S + offset, D]");
}

}  // namespace

std::tuple<at::Tensor, at::Tensor, at::Tensor> rope_qkv_forward(const at::Tensor& qkv, const at::Tensor& cos_t, const at::Tensor& sin_t,
                                                                int64_t offset) {
    TORCH_CHECK(qkv.is_cuda() && qkv.dim() == 5 && qkv.size(3) == 3 && qkv.is_contiguous(), "rope_qkv: contiguous CUDA [N, S, H, 3, D] required");
    TORCH_CHECK(qkv.scalar_type() == at::kBFloat16 || qkv.scalar_type() == at::kHalf, "rope_qkv: bf16 or fp16 required");
    const int64_t N = qkv.size(0), S = qkv.size(1), H = qkv.size(2), D = qkv.size(4);
    TORCH_CHECK(D % 16 == 0, "rope_qkv: head dimension must be a multiple of 16");
    check_tables(cos_t, sin_t, S, D, offset);
    const c10::cuda::CUDAGuard guard(qkv.device());
    at::Tensor q = at::empty({N, S, H, D}, qkv.options()), k = at::empty_like(q), v = at::empty_like(q);
    const long long rows = N * S * H, work = rows * (D / 2 / V);
    if (work == 0) return {q, k, v};
    const unsigned blocks = (unsigned)((work + 255) / 256);
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    if (qkv.scalar_type() == at::kBFloat16) {
        using T = __nv_bfloat16;
        rope_qkv_kernel<T, 1, false><<<blocks, 256, 0, st>>>(reinterpret_cast<const T*>(qkv.data_ptr()), nullptr, nullptr, nullptr, nullptr,
            reinterpret_cast<T*>(q.data_ptr()), reinterpret_cast<T*>(k.data_ptr()), reinterpret_cast<T*>(v.data_ptr()),
            cos_t.data_ptr<float>(), sin_t.data_ptr<float>(), rows, (int)S, (int)H, (int)D, (int)offset);
    } else {
        using T = __half;
        rope_qkv_kernel<T, 1, false><<<blocks, 256, 0, st>>>(reinterpret_cast<const T*>(qkv.data_ptr()), nullptr, nullptr, nullptr, nullptr,
            reinterpret_cast<T*>(q.data_ptr()), reinterpret_cast<T*>(k.data_ptr()), reinterpret_cast<T*>(v.data_ptr()),
            cos_t.data_ptr<float>(), sin_t.data_ptr<float>(), rows, (int)S, (int)H, (int)D, (int)offset);
    }
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return {q, k, v};
}

// gq, gk, gv: [N, S, H, D] contiguous -> gradient of the packed tensor [N, S, H, 3, D]
at::Tensor rope_qkv_backward(const at::Tensor& gq, const at::Tensor& gk, const at::Tensor& gv, const at::Tensor& cos_t,
                             const at::Tensor& sin_t, int64_t offset) {
    TORCH_CHECK(gq.is_cuda() && gq.dim() == 4 && gq.is_contiguous() && gk.is_contiguous() && gv.is_contiguous() &&
                gq.sizes() == gk.sizes() && gq.sizes() == gv.sizes() && gq.scalar_type() == gk.scalar_type() &&
                gq.scalar_type() == gv.scalar_type(), "rope_qkv_backward: three contiguous [N, S, H, D] tensors of one dtype required");
    TORCH_CHECK(gq.scalar_type() == at::kBFloat16 || gq.scalar_type() == at::kHalf, "rope_qkv_backward: bf16 or fp16 required");
    const int64_t N = gq.size(0), S = gq.size(1), H = gq.size(2), D = gq.size(3);
    check_tables(cos_t, sin_t, S, D, offset);
    const c10::cuda::CUDAGuard guard(gq.device());
    at::Tensor g = at::empty({N, S, H, 3, D}, gq.options());
    const long long rows = N * S * H, work = rows * (D / 2 / V);
    if (work == 0) return g;
    const unsigned blocks = (unsigned)((work + 255) / 256);
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    if (gq.scalar_type() == at::kBFloat16) {
        using T = __nv_bfloat16;
        rope_qkv_kernel<T, -1, true><<<blocks, 256, 0, st>>>(nullptr, reinterpret_cast<T*>(g.data_ptr()), reinterpret_cast<const T*>(gq.data_ptr()),
            reinterpret_cast<const T*>(gk.data_ptr()), reinterpret_cast<const T*>(gv.data_ptr()), nullptr, nullptr, nullptr,
            cos_t.data_ptr<float>(), sin_t.data_ptr<float>(), rows, (int)S, (int)H, (int)D, (int)offset);
    } else {
        using T = __half;
        rope_qkv_kernel<T, -1, true><<<blocks, 256, 0, st>>>(nullptr, reinterpret_cast<T*>(g.data_ptr()), reinterpret_cast<const T*>(gq.data_ptr()),
            reinterpret_cast<const T*>(gk.data_ptr()), reinterpret_cast<const T*>(gv.data_ptr()), nullptr, nullptr, nullptr,
            cos_t.data_ptr<float>(), sin_t.data_ptr<float>(), rows, (int)S, (int)H, (int)D, (int)offset);
    }
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return g;
}

}  // namespace sjb200

TORCH_LIBRARY_FRAGMENT(sjb200, m) {
    m.def("rope_qkv_forward(Tensor qkv, Tensor cos, Tensor sin, int offset) -> (Tensor, Tensor, Tensor)");
    m.def("rope_qkv_backward(Tensor gq, Tensor gk, Tensor gv, Tensor cos, Tensor sin, int offset) -> Tensor");
}
TORCH_LIBRARY_IMPL(sjb200, CUDA, m) {
    m.impl("rope_qkv_forward", &sjb200::rope_qkv_forward);
    m.impl("rope_qkv_backward", &sjb200::rope_qkv_backward);
}
