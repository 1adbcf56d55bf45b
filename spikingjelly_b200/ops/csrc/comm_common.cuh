// Peer-memory primitives shared by the collective kernels: the table of peer pointers, system-scope
// release/acquire accesses and the bounded flag barrier.  Peer data is only ever touched with plain ld/st
// (or multimem.* through the switch).
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
__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Flag comparison on full 32-bit wrapping counters: "flag has reached epoch".  The host wraps the epoch counter
// modulo 2^32 (never modulo 2^31), so the signed distance stays meaningful across the wrap.
__host__ __device__ __forceinline__ bool epoch_reached(uint32_t flag, uint32_t epoch) {
    return (int32_t)(flag - epoch) >= 0;
}

// Signal every peer and wait for every peer; threads 0..world-1 of the block take one peer each.
// The wait is bounded twice: by wall time (`timeout_ns` on the global timer, sampled every 1024 polls) and by an
// iteration count derived from it, so it ends even if the timer stood still.  Returns true (to every thread of
// the block) iff all peers arrived; on expiry {phase, peer} goes to the status word and the caller must not touch
// peer data.
__device__ __forceinline__ bool block_barrier(const PeerPtrs& pp, int rank, int world, int nblocks, uint32_t epoch,
                                              int phase, CommStatus* status, long long timeout_ns) {
    __syncthreads();
    bool ok = true;
    if ((int)threadIdx.x < world) {
        const int peer = threadIdx.x;
        // my slot on the peer: [block][rank]
        st_release_sys(pp.sig[peer] + (size_t)blockIdx.x * world + rank, epoch);
        const uint32_t* mine = pp.sig[rank] + (size_t)blockIdx.x * world + peer;
        const long long max_polls = timeout_ns / 16 + (1 << 16);
        unsigned long long t0 = 0;
        ok = false;
        for (long long i = 0; i < max_polls; ++i) {
            if (epoch_reached(ld_acquire_sys(mine), epoch)) { ok = true; break; }
            if (i > 32) {
                __nanosleep(i > 4096 ? 256 : 32);
                if ((i & 1023) == 0) {
                    const unsigned long long now = globaltimer_ns();
                    if (t0 == 0) t0 = now;
                    else if ((long long)(now - t0) > timeout_ns) break;
                }
            }
        }
        if (!ok && atomicCAS(&status->code, 0, phase) == 0) {
            status->rank = rank; status->peer = peer; status->block = blockIdx.x;
        }
    }
    return __syncthreads_and(ok) != 0;
}

}  // namespace comm
}  // namespace sjb200
