// Gradient-bucket all-reduce over NVLink peer memory, fused with the 1/world scaling (and an
// optional cast of the reduced result), as ONE kernel per bucket.
//
// Every rank owns a bucket of identical size in symmetric memory (each rank can address every
// peer's bucket).  Rank r reduces slice r of the bucket:
//     acc = sum over ranks j of bucket_j[slice_r]        (peer loads, or one in-switch
//                                                          multimem.ld_reduce when a multicast
//                                                          mapping exists)
//     bucket_j[slice_r] = acc * scale   for every j      (peer stores / multimem.st)
// i.e. reduce-scatter + all-gather in a single launch, with no intermediate buffer.
//
// Synchronisation: flags in a symmetric signal pad.  Block b of rank i signals slot
// [b][i] of every peer with a monotonically increasing epoch (release, system scope) and waits
// for the same epoch from every peer (acquire).  Phase 1 ("peer's bucket is complete": stream
// order on the peer guarantees that its gradient kernels finished before its all-reduce kernel
// started) precedes the loads; phase 2 ("all peers have written my slices") precedes kernel exit.
// Every wait is bounded: on expiry the block records {phase, peer} in a status word and carries
// on, so a missing peer yields an error code on the host instead of a hung GPU.
//
// Cluster-wide TMA loads are not used anywhere in this file: peer data moves with plain
// ld/st (or multimem), as required for kernels that touch another GPU's memory.
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

// fp32 buckets.  n4 = number of float4 in the bucket; slice of rank r: [r * per, min(n4, (r+1) * per))
__global__ void __launch_bounds__(kThreads)
allreduce_f32_kernel(PeerPtrs pp, int rank, int world, long long n4, float scale, uint32_t epoch, CommStatus* status,
                     long long spin_limit) {
    block_barrier(pp, rank, world, gridDim.x, epoch, 1, status, spin_limit);
    const long long per = (n4 + world - 1) / world;
    const long long lo = per * rank, hi = (lo + per < n4) ? lo + per : n4;
    for (long long i = lo + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < hi; i += (long long)gridDim.x * blockDim.x) {
        float4 v[kMaxWorld];
#pragma unroll
        for (int j = 0; j < kMaxWorld; ++j)
            if (j < world) v[j] = reinterpret_cast<const float4*>(pp.buf[j])[i];
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int j = 0; j < kMaxWorld; ++j)
            if (j < world) { acc.x += v[j].x; acc.y += v[j].y; acc.z += v[j].z; acc.w += v[j].w; }
        acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
#pragma unroll
        for (int j = 0; j < kMaxWorld; ++j)
            if (j < world) reinterpret_cast<float4*>(pp.buf[j])[i] = acc;
    }
    __threadfence_system();
    block_barrier(pp, rank, world, gridDim.x, epoch + 1, 2, status, spin_limit);
}

// Same exchange through the NVSwitch: one multimem.ld_reduce sums the slice across all ranks inside
// the switch, one multimem.st broadcasts the scaled result.  `mc` is the multicast mapping of the bucket.
__global__ void __launch_bounds__(kThreads)
allreduce_f32_multimem_kernel(PeerPtrs pp, float* mc, int rank, int world, long long n4, float scale, uint32_t epoch,
                              CommStatus* status, long long spin_limit) {
    block_barrier(pp, rank, world, gridDim.x, epoch, 1, status, spin_limit);
    const long long per = (n4 + world - 1) / world;
    const long long lo = per * rank, hi = (lo + per < n4) ? lo + per : n4;
    for (long long i = lo + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < hi; i += (long long)gridDim.x * blockDim.x) {
        float4 a;
        float* p = mc + i * 4;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                     : "=f"(a.x), "=f"(a.y), "=f"(a.z), "=f"(a.w) : "l"(p) : "memory");
        a.x *= scale; a.y *= scale; a.z *= scale; a.w *= scale;
        asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                     ::"l"(p), "f"(a.x), "f"(a.y), "f"(a.z), "f"(a.w) : "memory");
    }
    __threadfence_system();
    block_barrier(pp, rank, world, gridDim.x, epoch + 1, 2, status, spin_limit);
}

}  // namespace

// buf_ptrs / sig_ptrs: device addresses (as int64) of every rank's bucket and signal pad, index = rank.
// The signal pad must hold at least blocks * world uint32 and start zeroed; `epoch` must grow by 2 per call
// (the Python wrapper keeps the counter).  status: int32[4] on this device.
void allreduce_bucket(at::Tensor bucket, std::vector<int64_t> buf_ptrs, std::vector<int64_t> sig_ptrs, int64_t multicast_ptr,
                      int64_t rank, int64_t epoch, double scale, int64_t blocks, at::Tensor status, double timeout_s) {
    TORCH_CHECK(bucket.is_cuda() && bucket.is_contiguous() && bucket.scalar_type() == at::kFloat, "allreduce_bucket: contiguous fp32 CUDA bucket required");
    const int world = (int)buf_ptrs.size();
    TORCH_CHECK(world >= 1 && world <= kMaxWorld && (int)sig_ptrs.size() == world, "allreduce_bucket: bad world size");
    TORCH_CHECK(bucket.numel() % 4 == 0, "allreduce_bucket: bucket length must be a multiple of 4 floats");
    TORCH_CHECK(reinterpret_cast<uintptr_t>(bucket.data_ptr()) % 16 == 0, "allreduce_bucket: bucket must be 16-byte aligned");
    TORCH_CHECK(status.is_cuda() && status.scalar_type() == at::kInt && status.numel() >= 4, "allreduce_bucket: status must be int32[4]");
    const c10::cuda::CUDAGuard guard(bucket.device());
    PeerPtrs pp{};
    for (int j = 0; j < world; ++j) {
        pp.buf[j] = reinterpret_cast<void*>(buf_ptrs[j]);
        pp.sig[j] = reinterpret_cast<uint32_t*>(sig_ptrs[j]);
    }
    const long long n4 = bucket.numel() / 4;
    // ~100 ns per poll once the back-off is active
    const long long spin_limit = (long long)(timeout_s * 1e7) + 1000;
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    CommStatus* sp = reinterpret_cast<CommStatus*>(status.data_ptr<int>());
    if (multicast_ptr != 0) {
        allreduce_f32_multimem_kernel<<<(unsigned)blocks, kThreads, 0, st>>>(pp, reinterpret_cast<float*>(multicast_ptr), (int)rank, world, n4,
                                                                            (float)scale, (uint32_t)epoch, sp, spin_limit);
    } else {
        allreduce_f32_kernel<<<(unsigned)blocks, kThreads, 0, st>>>(pp, (int)rank, world, n4, (float)scale, (uint32_t)epoch, sp, spin_limit);
    }
    C10_CUDA_KERNEL_LAUNCH_CHECK();
}

}  // namespace sjb200

TORCH_LIBRARY_FRAGMENT(sjb200, m) {
    m.def("allreduce_bucket(Tensor(a!) bucket, int[] buf_ptrs, int[] sig_ptrs, int multicast_ptr, int rank, int epoch, "
          "float scale, int blocks, Tensor(b!) status, float timeout_s) -> ()");
}
TORCH_LIBRARY_IMPL(sjb200, CUDA, m) { m.impl("allreduce_bucket", &sjb200::allreduce_bucket); }
