// Peer-memory primitives shared by the collective kernels: the table of peer pointers, system-scope
// release/acquire accesses and the bounded flag barrier.  Peer data is only ever touched with plain ld/st.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace sjb200 {
namespace comm {

constexpr int kMaxWorld = 16;

struct PeerPtrs {
    void* buf[kMaxWorld];          // bucket base of every rank (peer-mapped)
    uint32_t* sig[kMaxWorld];      // signal pad of every rank
};

struct CommStatus { int code; int rank; int peer; int block; };   // code: 0 ok, 1 = phase-1 wait, 2 = phase-2 wait

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Signal every peer and wait for every peer; threads 0..world-1 of the block take one peer each.
__device__ __forceinline__ void block_barrier(const PeerPtrs& pp, int rank, int world, int nblocks, uint32_t epoch,
                                              int phase, CommStatus* status, long long spin_limit) {
    __syncthreads();
    if ((int)threadIdx.x < world) {
        const int peer = threadIdx.x;
        // my slot on the peer: [block][rank]
        st_release_sys(pp.sig[peer] + (size_t)blockIdx.x * world + rank, epoch);
        const uint32_t* mine = pp.sig[rank] + (size_t)blockIdx.x * world + peer;
        bool ok = false;
        for (long long i = 0; i < spin_limit; ++i) {
            if ((int32_t)(ld_acquire_sys(mine) - epoch) >= 0) { ok = true; break; }
            if (i > 32) __nanosleep(64);
        }
        if (!ok && atomicCAS(&status->code, 0, phase) == 0) {
            status->rank = rank; status->peer = peer; status->block = blockIdx.x;
        }
    }
    __syncthreads();
}

}  // namespace comm
}  // namespace sjb200
