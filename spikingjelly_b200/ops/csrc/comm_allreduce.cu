// Gradient-bucket all-reduce over NVLink peer memory, fused with the 1/world scaling and (optionally) a
// cast to a bf16 wire format, as ONE kernel per bucket.
//
// Every rank owns a bucket of identical size in symmetric memory (each rank can address every peer's
// bucket).  Rank r reduces slice r of the bucket:
//     acc = sum over ranks j of bucket_j[slice_r]        (peer loads, or one in-switch
//                                                          multimem.ld_reduce when a multicast
//                                                          mapping exists)
//     bucket_j[slice_r] = acc * scale   for every j      (peer stores / multimem.st)
// i.e. reduce-scatter + all-gather in a single launch, with no intermediate buffer.
//
// bf16 wire (`wire == 1`): the fp32 bucket stays the master copy, but what crosses NVLink is bf16.  The
// kernel first casts the local bucket into a bf16 staging buffer (symmetric memory as well), reduces the
// staging slices with fp32 accumulation, writes the scaled bf16 result into every rank's staging buffer and
// finally widens the local staging buffer back into the fp32 bucket.  The cast and the widening use the same
// (block, thread) -> element mapping as the exchange, so a block only depends on the SAME block index of
// each peer and the per-block flag barrier is sufficient.
//
// Synchronisation: flags in a symmetric signal pad.  Block b of rank i signals slot [b][i] of every peer
// with a monotonically increasing epoch (release, system scope) and waits for the same epoch from every
// peer (acquire).  Phase 1 ("peer's bucket is complete": stream order on the peer guarantees that its
// gradient kernels finished before its all-reduce kernel started) precedes the loads; phase 2 ("all peers
// have written my slices") precedes kernel exit.  Every wait is bounded in time: on expiry the block records
// {phase, peer} in a status word, SKIPS every access to peer memory (its slice stays un-reduced rather than
// becoming a sum of unfinished buckets, and nothing is stored into a peer that may still be running
// backward) and still signals phase 2 so that the peers do not wait for it in vain.  The host turns the
// status word into an exception.
//
// Cluster-wide TMA loads are not used anywhere in this file: peer data moves with plain ld/st (or
// multimem), as required for kernels that touch another GPU's memory.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <cuda_bf16.h>
#include <stdint.h>

#include "comm_common.cuh"

namespace sjb200 {
namespace {

using namespace comm;

constexpr int kThreads = 512;

// A thread keeps U x WMAX 16-byte loads in flight: over NVLink (a few microseconds of latency) the exchange is bound by
// the bytes in flight, not by the link, unless every thread has several independent loads outstanding.  WMAX bounds
// the world size of an instantiation (2, 4, 8 or 16); U is chosen so that U * WMAX stays near 8.
template <int WMAX> struct Unroll { static constexpr int U = WMAX <= 2 ? 4 : (WMAX <= 4 ? 2 : 1); };
constexpr int kMultimemUnroll = 8;

// ----------------------------------------------------------------------------------------------- fp32 wire
// n4 = number of float4 in the bucket; slice of rank r: [r * per, min(n4, (r+1) * per))
template <int WMAX>
__global__ void __launch_bounds__(kThreads)
allreduce_f32_kernel(PeerPtrs pp, int rank, int world, long long n4, float scale, uint32_t epoch, CommStatus* status,
                     long long timeout_ns) {
    constexpr int U = Unroll<WMAX>::U;
    const bool ok = block_barrier(pp, rank, world, gridDim.x, epoch, 1, status, timeout_ns);
    const long long per = (n4 + world - 1) / world;
    const long long lo = per * rank, hi = (lo + per < n4) ? lo + per : n4;
    const long long stride = (long long)gridDim.x * blockDim.x;
    if (ok) {
        for (long long i0 = lo + (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < hi; i0 += stride * U) {
            float4 v[U][WMAX];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const long long i = i0 + u * stride;
#pragma unroll
                for (int j = 0; j < WMAX; ++j)
                    if (j < world && i < hi) v[u][j] = reinterpret_cast<const float4*>(pp.buf[j])[i];
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const long long i = i0 + u * stride;
                if (i >= hi) break;
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int j = 0; j < WMAX; ++j)
                    if (j < world) { acc.x += v[u][j].x; acc.y += v[u][j].y; acc.z += v[u][j].z; acc.w += v[u][j].w; }
                acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
#pragma unroll
                for (int j = 0; j < WMAX; ++j)
                    if (j < world) reinterpret_cast<float4*>(pp.buf[j])[i] = acc;
            }
        }
    }
    __threadfence_system();
    block_barrier(pp, rank, world, gridDim.x, epoch + 1, 2, status, timeout_ns);
}

// Same exchange through the NVSwitch: one multimem.ld_reduce sums the slice across all ranks inside
// the switch, one multimem.st broadcasts the scaled result.  `mc` is the multicast mapping of the bucket.
__global__ void __launch_bounds__(kThreads)
allreduce_f32_multimem_kernel(PeerPtrs pp, float* mc, int rank, int world, long long n4, float scale, uint32_t epoch,
                              CommStatus* status, long long timeout_ns) {
    constexpr int U = kMultimemUnroll;
    const bool ok = block_barrier(pp, rank, world, gridDim.x, epoch, 1, status, timeout_ns);
    const long long per = (n4 + world - 1) / world;
    const long long lo = per * rank, hi = (lo + per < n4) ? lo + per : n4;
    const long long stride = (long long)gridDim.x * blockDim.x;
    if (ok) {
        for (long long i0 = lo + (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < hi; i0 += stride * U) {
            float4 a[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const long long i = i0 + u * stride;
                if (i < hi)
                    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                                 : "=f"(a[u].x), "=f"(a[u].y), "=f"(a[u].z), "=f"(a[u].w) : "l"(mc + i * 4) : "memory");
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const long long i = i0 + u * stride;
                if (i < hi)
                    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                                 ::"l"(mc + i * 4), "f"(a[u].x * scale), "f"(a[u].y * scale), "f"(a[u].z * scale), "f"(a[u].w * scale) : "memory");
            }
        }
    }
    __threadfence_system();
    block_barrier(pp, rank, world, gridDim.x, epoch + 1, 2, status, timeout_ns);
}

// ----------------------------------------------------------------------------------------------- bf16 wire
__device__ __forceinline__ uint4 pack8(const float* f) {
    uint4 r;
    __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int q = 0; q < 4; ++q) p[q] = __floats2bfloat162_rn(f[2 * q], f[2 * q + 1]);
    return r;
}
__device__ __forceinline__ void unpack8(const uint4& r, float* f) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
    for (int q = 0; q < 4; ++q) { const float2 t = __bfloat1622float2(p[q]); f[2 * q] = t.x; f[2 * q + 1] = t.y; }
}

// n8 = number of 8-element units in the bucket.  `stage` holds every rank's bf16 staging buffer (pp.buf) and
// `bucket` is this rank's fp32 master copy.  MULTIMEM: the slice exchange goes through the multicast mapping
// `mc` of the staging buffer.
template <bool MULTIMEM, int WMAX>
__global__ void __launch_bounds__(kThreads)
allreduce_bf16wire_kernel(PeerPtrs pp, float* bucket, __nv_bfloat16* mc, int rank, int world, long long n8,
                          float scale, uint32_t epoch, CommStatus* status, long long timeout_ns) {
    constexpr int UL = 4;                                   // local passes (cast, widen): units per thread and round
    const long long per = (n8 + world - 1) / world;
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long first = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    uint4* mine = reinterpret_cast<uint4*>(pp.buf[rank]);
    // cast: for every slice s, the units that block `blockIdx.x` of rank s will read
    for (int s = 0; s < world; ++s) {
        const long long lo = per * s, hi = (lo + per < n8) ? lo + per : n8;
        for (long long u0 = lo + first; u0 < hi; u0 += stride * UL) {
            float4 a[UL], b[UL];
#pragma unroll
            for (int k = 0; k < UL; ++k) {
                const long long u = u0 + k * stride;
                if (u < hi) { a[k] = reinterpret_cast<const float4*>(bucket)[2 * u]; b[k] = reinterpret_cast<const float4*>(bucket)[2 * u + 1]; }
            }
#pragma unroll
            for (int k = 0; k < UL; ++k) {
                const long long u = u0 + k * stride;
                if (u < hi) {
                    const float f[8] = {a[k].x, a[k].y, a[k].z, a[k].w, b[k].x, b[k].y, b[k].z, b[k].w};
                    mine[u] = pack8(f);
                }
            }
        }
    }
    __threadfence_system();
    const bool ok = block_barrier(pp, rank, world, gridDim.x, epoch, 1, status, timeout_ns);
    if (ok) {
        const long long lo = per * rank, hi = (lo + per < n8) ? lo + per : n8;
        if constexpr (MULTIMEM) {
            constexpr int U = kMultimemUnroll;
            for (long long u0 = lo + first; u0 < hi; u0 += stride * U) {
                uint4 r[U];
#pragma unroll
                for (int k = 0; k < U; ++k) {
                    const long long u = u0 + k * stride;
                    if (u < hi)
                        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                                     : "=r"(r[k].x), "=r"(r[k].y), "=r"(r[k].z), "=r"(r[k].w) : "l"(mc + u * 8) : "memory");
                }
#pragma unroll
                for (int k = 0; k < U; ++k) {
                    const long long u = u0 + k * stride;
                    if (u < hi) {
                        float acc[8];
                        unpack8(r[k], acc);
#pragma unroll
                        for (int q = 0; q < 8; ++q) acc[q] *= scale;
                        const uint4 o = pack8(acc);
                        asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};"
                                     ::"l"(mc + u * 8), "r"(o.x), "r"(o.y), "r"(o.z), "r"(o.w) : "memory");
                    }
                }
            }
        } else {
            constexpr int U = Unroll<WMAX>::U;
            for (long long u0 = lo + first; u0 < hi; u0 += stride * U) {
                uint4 v[U][WMAX];
#pragma unroll
                for (int k = 0; k < U; ++k) {
                    const long long u = u0 + k * stride;
#pragma unroll
                    for (int j = 0; j < WMAX; ++j)
                        if (j < world && u < hi) v[k][j] = reinterpret_cast<const uint4*>(pp.buf[j])[u];
                }
#pragma unroll
                for (int k = 0; k < U; ++k) {
                    const long long u = u0 + k * stride;
                    if (u >= hi) break;
                    float acc[8];
#pragma unroll
                    for (int q = 0; q < 8; ++q) acc[q] = 0.f;
#pragma unroll
                    for (int j = 0; j < WMAX; ++j)
                        if (j < world) {
                            float f[8];
                            unpack8(v[k][j], f);
#pragma unroll
                            for (int q = 0; q < 8; ++q) acc[q] += f[q];
                        }
#pragma unroll
                    for (int q = 0; q < 8; ++q) acc[q] *= scale;
                    const uint4 o = pack8(acc);
#pragma unroll
                    for (int j = 0; j < WMAX; ++j)
                        if (j < world) reinterpret_cast<uint4*>(pp.buf[j])[u] = o;
                }
            }
        }
    }
    __threadfence_system();
    const bool ok2 = block_barrier(pp, rank, world, gridDim.x, epoch + 1, 2, status, timeout_ns);
    if (ok && ok2) {
        // widen: the same units this block cast above; block `blockIdx.x` of rank s has written slice s of them
        for (int s = 0; s < world; ++s) {
            const long long lo = per * s, hi = (lo + per < n8) ? lo + per : n8;
            for (long long u0 = lo + first; u0 < hi; u0 += stride * UL) {
                uint4 r[UL];
#pragma unroll
                for (int k = 0; k < UL; ++k) {
                    const long long u = u0 + k * stride;
                    if (u < hi) r[k] = __ldcg(mine + u);      // the peers' stores arrived through NVLink: read around L1
                }
#pragma unroll
                for (int k = 0; k < UL; ++k) {
                    const long long u = u0 + k * stride;
                    if (u < hi) {
                        float f[8];
                        unpack8(r[k], f);
                        reinterpret_cast<float4*>(bucket)[2 * u] = make_float4(f[0], f[1], f[2], f[3]);
                        reinterpret_cast<float4*>(bucket)[2 * u + 1] = make_float4(f[4], f[5], f[6], f[7]);
                    }
                }
            }
        }
    }
}

}  // namespace

// buf_ptrs / sig_ptrs: device addresses (as int64) of every rank's exchange buffer and signal pad, index = rank.
// wire == 0: the exchange buffer IS the fp32 bucket.  wire == 1: the exchange buffer is a bf16 staging buffer of
// bucket.numel() elements in symmetric memory, the bucket itself is only touched locally.
// multicast_ptr: multicast mapping of the exchange buffer, or 0 for plain peer loads/stores.
// The signal pad must hold at least blocks * world uint32 and start zeroed; `epoch` must grow by 2 per call
// modulo 2^32 (the Python wrapper keeps the counter).  status: int32[4] on this device.
void allreduce_bucket(at::Tensor bucket, std::vector<int64_t> buf_ptrs, std::vector<int64_t> sig_ptrs, int64_t multicast_ptr,
                      int64_t rank, int64_t epoch, double scale, int64_t blocks, at::Tensor status, double timeout_s,
                      int64_t wire) {
    TORCH_CHECK(bucket.is_cuda() && bucket.is_contiguous() && bucket.scalar_type() == at::kFloat, "allreduce_bucket: contiguous fp32 CUDA bucket required");
    const int world = (int)buf_ptrs.size();
    TORCH_CHECK(world >= 1 && world <= kMaxWorld && (int)sig_ptrs.size() == world, "allreduce_bucket: bad world size");
    TORCH_CHECK(wire == 0 || wire == 1, "allreduce_bucket: wire must be 0 (fp32) or 1 (bf16)");
    TORCH_CHECK(bucket.numel() % (wire == 0 ? 4 : 8) == 0, "allreduce_bucket: bucket length must be a multiple of 4 (fp32 wire) / 8 (bf16 wire) elements");
    TORCH_CHECK(reinterpret_cast<uintptr_t>(bucket.data_ptr()) % 16 == 0, "allreduce_bucket: bucket must be 16-byte aligned");
    TORCH_CHECK(status.is_cuda() && status.scalar_type() == at::kInt && status.numel() >= 4, "allreduce_bucket: status must be int32[4]");
    TORCH_CHECK(blocks >= 1 && blocks <= 1024, "allreduce_bucket: bad block count");
    TORCH_CHECK(rank >= 0 && rank < world, "allreduce_bucket: bad rank");
    const c10::cuda::CUDAGuard guard(bucket.device());
    PeerPtrs pp{};
    for (int j = 0; j < world; ++j) {
        TORCH_CHECK(buf_ptrs[j] % 16 == 0, "allreduce_bucket: exchange buffers must be 16-byte aligned");
        pp.buf[j] = reinterpret_cast<void*>(buf_ptrs[j]);
        pp.sig[j] = reinterpret_cast<uint32_t*>(sig_ptrs[j]);
    }
    const long long timeout_ns = (long long)(timeout_s * 1e9) + 1000;
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    CommStatus* sp = reinterpret_cast<CommStatus*>(status.data_ptr<int>());
    const unsigned g = (unsigned)blocks;
#define SJ_BY_WORLD(CALL)                      \
    do {                                       \
        if (world <= 2) { CALL(2); }           \
        else if (world <= 4) { CALL(4); }      \
        else if (world <= 8) { CALL(8); }      \
        else { CALL(16); }                     \
    } while (0)
    if (wire == 0) {
        TORCH_CHECK(buf_ptrs[rank] == reinterpret_cast<int64_t>(bucket.data_ptr()), "allreduce_bucket: buf_ptrs[rank] must be the bucket itself for the fp32 wire");
        const long long n4 = bucket.numel() / 4;
        if (multicast_ptr != 0) {
            allreduce_f32_multimem_kernel<<<g, kThreads, 0, st>>>(pp, reinterpret_cast<float*>(multicast_ptr), (int)rank, world, n4,
                                                                  (float)scale, (uint32_t)epoch, sp, timeout_ns);
        } else {
#define SJ_CALL(W) allreduce_f32_kernel<W><<<g, kThreads, 0, st>>>(pp, (int)rank, world, n4, (float)scale, (uint32_t)epoch, sp, timeout_ns)
            SJ_BY_WORLD(SJ_CALL);
#undef SJ_CALL
        }
    } else {
        const long long n8 = bucket.numel() / 8;
        if (multicast_ptr != 0) {
            allreduce_bf16wire_kernel<true, 2><<<g, kThreads, 0, st>>>(pp, bucket.data_ptr<float>(), reinterpret_cast<__nv_bfloat16*>(multicast_ptr),
                                                                       (int)rank, world, n8, (float)scale, (uint32_t)epoch, sp, timeout_ns);
        } else {
#define SJ_CALL(W) allreduce_bf16wire_kernel<false, W><<<g, kThreads, 0, st>>>(pp, bucket.data_ptr<float>(), nullptr, (int)rank, world, n8, \
                                                                              (float)scale, (uint32_t)epoch, sp, timeout_ns)
            SJ_BY_WORLD(SJ_CALL);
#undef SJ_CALL
        }
    }
#undef SJ_BY_WORLD
    C10_CUDA_KERNEL_LAUNCH_CHECK();
}

}  // namespace sjb200

TORCH_LIBRARY_FRAGMENT(sjb200, m) {
    m.def("allreduce_bucket(Tensor(a!) bucket, int[] buf_ptrs, int[] sig_ptrs, int multicast_ptr, int rank, int epoch, "
          "float scale, int blocks, Tensor(b!) status, float timeout_s, int wire=0) -> ()");
}
TORCH_LIBRARY_IMPL(sjb200, CUDA, m) { m.impl("allreduce_bucket", &sjb200::allreduce_bucket); }
