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
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdlib>
#include <torch/library.h>

#include "tc_common.cuh"
#include "tma_host.cuh"

namespace sjb200 {
namespace {

using namespace tc;

constexpr int BM = 128;
constexpr int BK = 64;          // 64 x 2 B = one 128 B swizzle row
constexpr int UMMA_K = 16;
constexpr int kThreads = 320;   // 10 warps: producer, mma, 2 x 4 epilogue (each group of four drains half of the columns)

template <int BN, int STAGES>
struct SmemLayout {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
    static constexpr int OUT_OFFSET = BAR_OFFSET + 1024;    // epilogue staging: 2 groups x 2 x [128 rows][32 cols] 16-bit
    static constexpr int OUT_BYTES = BM * 32 * 2;
    static constexpr int TOTAL = OUT_OFFSET + 4 * OUT_BYTES + 1024;   // + slack for 1024 B alignment
};

// Output tiles are visited in column groups of kGroupN tiles: within a group all row tiles are visited (n fastest), so
// the CTAs that run together share kGroupN column tiles of B (they stay in L2 for the whole group) and a few row
// tiles of A.  With plain n-fastest order a wide B (N * K * 2 B beyond the L2 size) is re-read from DRAM once per
// row of tiles.
constexpr int kGroupN = 8;
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
    const int per_group = tiles_m * kGroupN;
    const int grp = t / per_group, in = t - grp * per_group;
    const int gw = min(kGroupN, tiles_n - grp * kGroupN);
    tm = in / gw;
    tn = grp * kGroupN + (in - tm * gw);
}

struct GemmArgs {
    int M, N, K;            // logical sizes (K = contraction)
    int ldd;                // leading dimension of D (elements)
    int split_k;            // >= 1
    int kb_per_split;       // k-blocks (of BK) per split
    int out_f32;            // D is fp32 (always when split_k > 1)
    int ab_format;          // kind::f16: 0 = fp16, 1 = bf16;  kind::f8f6f4: 0 = e4m3, 1 = e5m2 (A and B alike)
    int out_bf16;           // 16-bit results are bf16 (else fp16)
    const float* alpha;     // optional device scalar multiplied into the result (product of the fp8 scales)
    float* stats;           // optional [ceil(M / 128) * 4][2][N]: per-column sum and sum of squares of the rounded
                            // 16-bit result over each 32-row slice (batch-norm statistics without re-reading D)
};

// ES: operand element size in bytes (2: fp16 / bf16, 1: fp8).  A k-block is always one 128-byte
// swizzle row, i.e. 128 / ES elements, and is consumed by four MMAs of 32 bytes of K each.
template <int BN, int STAGES, bool A_MN, bool B_MN, int ES = 2>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ CUtensorMap tmD, void* __restrict__ Dptr, GemmArgs g, KernelStatus* __restrict__ status) {
    using L = SmemLayout<BN, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* tfull_bar = empty_bar + STAGES;
    uint64_t* tempty_bar = tfull_bar + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (g.M + BM - 1) / BM, tiles_n = (g.N + BN - 1) / BN;
    const int tiles_mn = tiles_m * tiles_n;
    const int total_tiles = tiles_mn * g.split_k;
    constexpr int BKE = 128 / ES;              // elements per k-block
    static_assert(ES == 2 || (!A_MN && !B_MN), "8-bit operands are K-major only");
    const int kb_total = (g.K + BKE - 1) / BKE;
    const float alpha = g.alpha != nullptr ? __ldg(g.alpha) : 1.0f;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar + s, 1); mbar_init(empty_bar + s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar + a, 1); mbar_init(tempty_bar + a, 8); }
        *abort_flag = 0;
        mbar_init_fence();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 2 * BN);
        tmem_relinquish();
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t it = 0;
            for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x) {
                const int split = tile / tiles_mn, mn = tile % tiles_mn;
                int tm, tn;
                tile_coords(mn, tiles_m, tiles_n, tm, tn);
                const int m0 = tm * BM, n0 = tn * BN;
                const int kb0 = split * g.kb_per_split;
                const int kb1 = min(kb_total, kb0 + g.kb_per_split);
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait_bounded(empty_bar + s, ph ^ 1)) { report(status, WAIT_EMPTY, s); *abort_flag = 1; break; }
                    uint8_t* sa = smem + s * L::STAGE_BYTES;
                    uint8_t* sb = sa + L::A_BYTES;
                    mbar_expect_tx(full_bar + s, L::STAGE_BYTES);
                    const int k0 = kb * BKE;
                    if (A_MN) {
#pragma unroll
                        for (int c = 0; c < BM / 64; ++c) tma_load_2d(sa + c * (BK * 128), &tmA, m0 + c * 64, k0, full_bar + s);
                    } else {
                        tma_load_2d(sa, &tmA, k0, m0, full_bar + s);
                    }
                    if (B_MN) {
#pragma unroll
                        for (int c = 0; c < BN / 64; ++c) tma_load_2d(sb + c * (BK * 128), &tmB, n0 + c * 64, k0, full_bar + s);
                    } else {
                        tma_load_2d(sb, &tmB, k0, n0, full_bar + s);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            const uint32_t idesc = make_idesc_f16(g.ab_format, A_MN ? 1 : 0, B_MN ? 1 : 0, BM, BN);
            uint32_t it = 0, tl = 0;
            for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x, ++tl) {
                const int split = tile / tiles_mn;
                const int kb0 = split * g.kb_per_split;
                const int kb1 = min(kb_total, kb0 + g.kb_per_split);
                const uint32_t acc = tl & 1, acc_ph = (tl >> 1) & 1;
                if (!mbar_wait_bounded(tempty_bar + acc, acc_ph ^ 1)) { report(status, WAIT_TMEM_EMPTY, tile); *abort_flag = 1; break; }
                fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait_bounded(full_bar + s, ph)) { report(status, WAIT_FULL, s); *abort_flag = 1; break; }
                    fence_after_sync();
                    const uint32_t sa = smem_u32(smem + s * L::STAGE_BYTES);
                    const uint32_t sb = sa + L::A_BYTES;
#pragma unroll
                    for (int j = 0; j < BK / UMMA_K; ++j) {
                        // K-major: 16 elements = 32 B further along the swizzled row;
                        // MN-major: 16 k-rows of 128 B further down.
                        const uint64_t da = A_MN ? make_smem_desc(sa + j * (UMMA_K * 128), BK * 128, 1024)
                                                 : make_smem_desc(sa + j * (UMMA_K * 2), 16, 1024);
                        const uint64_t db = B_MN ? make_smem_desc(sb + j * (UMMA_K * 128), BK * 128, 1024)
                                                 : make_smem_desc(sb + j * (UMMA_K * 2), 16, 1024);
                        if constexpr (ES == 2) mma_f16_ss(d_tmem, da, db, idesc, (kb > kb0 || j > 0) ? 1u : 0u);
                        else mma_f8_ss(d_tmem, da, db, idesc, (kb > kb0 || j > 0) ? 1u : 0u);
                    }
                    mma_commit(empty_bar + s);     // stage reusable once these MMAs have read it
                }
                mma_commit(tfull_bar + acc);       // accumulator complete
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        const int quarter = warp & 3;              // TMEM lane quarter this warp may read
        const int half = (warp - 2) >> 2;          // which half of the tile's columns this group of four warps drains
        const int issuer = 64 + half * 128;        // the thread of the group that talks to the TMA unit
        uint32_t tl = 0, oc = 0;                   // tiles / output chunks handled so far
        for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x, ++tl) {
            const int split = tile / tiles_mn, mn = tile % tiles_mn;
            int tm, tn;
            tile_coords(mn, tiles_m, tiles_n, tm, tn);
            const int m0 = tm * BM, n0 = tn * BN;
            const uint32_t acc = tl & 1, acc_ph = (tl >> 1) & 1;
            bool ok = true;
            if (lane == 0) ok = mbar_wait_bounded(tfull_bar + acc, acc_ph);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) { if (lane == 0) { report(status, WAIT_TMEM_FULL, tile); *abort_flag = 1; } break; }
            fence_after_sync();
            const int row = m0 + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
#pragma unroll 1
            for (int c = half * (BN / 64); c < (half + 1) * (BN / 64); ++c) {
                uint32_t r[32];
                tmem_ld_32x32(taddr + c * 32, r);
                tmem_ld_wait();
                if (g.alpha != nullptr) {
#pragma unroll
                    for (int q = 0; q < 32; ++q) r[q] = __float_as_uint(__uint_as_float(r[q]) * alpha);
                }
                const int col0 = n0 + c * 32;
                if (row < g.M && col0 < g.N) {
                    if (g.out_f32) {
                        float* dst = reinterpret_cast<float*>(Dptr) + ((size_t)split * g.M + row) * g.ldd + col0;
                        if (col0 + 32 <= g.N) {
#pragma unroll
                            for (int q = 0; q < 8; ++q)
                                reinterpret_cast<uint4*>(dst)[q] = make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
                        } else {
#pragma unroll
                            for (int q = 0; q < 32; ++q)
                                if (col0 + q < g.N) dst[q] = __uint_as_float(r[q]);
                        }
                    }
                }
                if (!g.out_f32) {
                    // 16-bit output: stage the 128 x 32 chunk in shared memory (64-byte rows, 16-byte
                    // chunks XOR-swizzled by (row >> 1) & 3 = the TMA 64B swizzle) and let TMA write it:
                    // full-sector, clipped at the matrix edges, asynchronous.
                    uint8_t* stage_buf = smem + L::OUT_OFFSET + (half * 2 + (oc & 1)) * L::OUT_BYTES;
                    if (oc >= 2 && (int)threadIdx.x == issuer) tma_store_wait_read<1>();  // the store that last read this buffer is done
                    ++oc;
                    named_barrier(1 + half, 128);
                    const int r_in_tile = quarter * 32 + lane;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        uint32_t w[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float lo = __uint_as_float(r[8 * q + 2 * e]), hi = __uint_as_float(r[8 * q + 2 * e + 1]);
                            if (g.out_bf16) { __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi); w[e] = *reinterpret_cast<uint32_t*>(&v); }
                            else { __half2 v = __floats2half2_rn(lo, hi); w[e] = *reinterpret_cast<uint32_t*>(&v); }
                        }
                        const int chunk = q ^ ((r_in_tile >> 1) & 3);
                        *reinterpret_cast<uint4*>(stage_buf + r_in_tile * 64 + chunk * 16) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                    fence_async_smem();
                    named_barrier(1 + half, 128);
                    if ((int)threadIdx.x == issuer) {
                        tma_store_2d(&tmD, stage_buf, n0 + c * 32, m0);
                        tma_store_commit();
                    }
                    if (g.stats != nullptr) {
                        // Column sums over this warp's own 32 staged rows (the rounded values BN will read).
                        // Lane = (column pair, row half); the upper half walks its rows one step ahead so that the
                        // two halves hit different 64-byte halves of a bank line.
                        const int cp = lane & 15, hi = lane >> 4;
                        float s1a = 0.f, s1b = 0.f, s2a = 0.f, s2b = 0.f;
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const int rr = quarter * 32 + hi * 16 + ((i + hi) & 15);
                            const int chunk = (cp >> 2) ^ ((rr >> 1) & 3);
                            const uint32_t w = *reinterpret_cast<const uint32_t*>(stage_buf + rr * 64 + chunk * 16 + (cp & 3) * 4);
                            float lo, up;
                            if (g.out_bf16) { lo = __uint_as_float(w << 16); up = __uint_as_float(w & 0xffff0000u); }
                            else { const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w)); lo = f.x; up = f.y; }
                            s1a += lo; s1b += up; s2a = fmaf(lo, lo, s2a); s2b = fmaf(up, up, s2b);
                        }
                        s1a += __shfl_xor_sync(0xffffffffu, s1a, 16); s1b += __shfl_xor_sync(0xffffffffu, s1b, 16);
                        s2a += __shfl_xor_sync(0xffffffffu, s2a, 16); s2b += __shfl_xor_sync(0xffffffffu, s2b, 16);
                        const int col = n0 + c * 32 + cp * 2;
                        if (hi == 0 && col < g.N) {
                            float* dst = g.stats + ((size_t)((m0 / BM) * 4 + quarter) * 2) * g.N + col;
                            *reinterpret_cast<float2*>(dst) = make_float2(s1a, s1b);
                            *reinterpret_cast<float2*>(dst + g.N) = make_float2(s2a, s2b);
                        }
                    }
                }
            }
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar + acc);
        }
        if ((int)threadIdx.x == issuer) tma_store_wait_all<0>();   // all output boxes written before the CTA retires
    }

    // -------------------------------------------------------------------- teardown
    if (*abort_flag) {
        // let copies that are still in flight land before the CTA's shared memory goes away
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    if (warp == 1) tmem_dealloc(tmem_base, 2 * BN);
}

// ---- CTA-pair variant -----------------------------------------------------------------------------------
// Two CTAs of a cluster (two SMs) work on one 256 x 256 output tile.  Each CTA loads 128 rows of A and 128 of the 256
// columns' worth of B per k-block (32 KB instead of the 48 KB a 128 x 256 single-CTA tile needs for half the
// output), one thread of the pair's first CTA issues `tcgen05.mma.cta_group::2` (M = 256, N = 256), and each CTA ends
// up with its 128 rows x 256 columns of the accumulator in its own TMEM, which its own epilogue warps drain.
// Barrier protocol:
//   full[s]   (first CTA only)  expect 2 x 32 KB: both producers' TMA loads credit it
//   empty[s]  (each CTA)        one arrival per round: the MMA thread commits to the local and to the peer's barrier
//   tfull[a]  (each CTA)        likewise, after the last k-block of a tile
//   tempty[a] (first CTA only)  16 arrivals: the 8 epilogue warps of both CTAs
// Cluster barriers bracket the kernel: nobody signals into a CTA whose barriers are not initialised yet, and no CTA
// retires (or frees tensor memory) while its partner may still read its shared memory or write its TMEM.
constexpr int kPairStages = 6;
constexpr int kPairBN = 256;
struct PairSmem {
    static constexpr int A_BYTES = BM * BK * 2;                 // this CTA's 128 rows of A
    static constexpr int B_BYTES = (kPairBN / 2) * BK * 2;      // this CTA's 128 of the 256 columns of B
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int BAR_OFFSET = kPairStages * STAGE_BYTES;
    static constexpr int OUT_OFFSET = BAR_OFFSET + 1024;
    static constexpr int OUT_BYTES = BM * 32 * 2;
    static constexpr int TOTAL = OUT_OFFSET + 4 * OUT_BYTES + 1024;
};

template <bool A_MN, bool B_MN, int ES = 2>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmD, void* __restrict__ Dptr, GemmArgs g, KernelStatus* __restrict__ status) {
    static_assert(ES == 2 || (!A_MN && !B_MN), "8-bit operands are K-major only");
    constexpr int BKE = 128 / ES;                            // elements per k-block (one 128-byte swizzle row)
    using L = PairSmem;
    constexpr int STAGES = kPairStages, BN = kPairBN;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* tfull_bar = empty_bar + STAGES;
    uint64_t* tempty_bar = tfull_bar + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();                 // 0: issues the MMAs; 1: partner
    const bool first = rank == 0;
    const int tiles_m = (g.M + 2 * BM - 1) / (2 * BM), tiles_n = (g.N + BN - 1) / BN;
    const int tiles_mn = tiles_m * tiles_n;
    const int total_tiles = tiles_mn * g.split_k;
    const int pair = (int)blockIdx.x >> 1, n_pairs = (int)gridDim.x >> 1;
    const int kb_total = (g.K + BKE - 1) / BKE;
    const float alpha = g.alpha != nullptr ? __ldg(g.alpha) : 1.0f;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar + s, 1); mbar_init(empty_bar + s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar + a, 1); mbar_init(tempty_bar + a, 16); }
        *abort_flag = 0;
        mbar_init_fence();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
    }
    __syncthreads();
    cluster_sync_all();                                      // both CTAs' barriers exist before anyone signals them
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, 2 * BN);
        tmem_relinquish_pair();
    }
    fence_before_sync();
    __syncthreads();
    cluster_sync_all();                                      // both halves of the accumulator are allocated
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (one thread in each CTA)
        if (lane == 0) {
            uint32_t it = 0;
            for (int tile = pair; tile < total_tiles && !*abort_flag; tile += n_pairs) {
                const int split = tile / tiles_mn;
                int tm, tn;
                tile_coords(tile - split * tiles_mn, tiles_m, tiles_n, tm, tn);
                const int m0 = tm * (2 * BM) + (int)rank * BM;
                const int nb0 = tn * BN + (int)rank * (BN / 2);                    // this CTA's half of the B columns
                const int kb0 = split * g.kb_per_split, kb1 = min(kb_total, kb0 + g.kb_per_split);
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait_bounded(empty_bar + s, ph ^ 1)) { report(status, WAIT_EMPTY, s); *abort_flag = 1; break; }
                    uint8_t* sa = smem + s * L::STAGE_BYTES;
                    uint8_t* sb = sa + L::A_BYTES;
                    if (first) mbar_expect_tx(full_bar + s, 2 * L::STAGE_BYTES);
                    const uint32_t bar = map_to_cta(smem_u32(full_bar + s), 0);
                    const int k0 = kb * BKE;
                    if (A_MN) {
#pragma unroll
                        for (int c = 0; c < BM / 64; ++c) tma_load_2d_pair(sa + c * (BK * 128), &tmA, m0 + c * 64, k0, bar);
                    } else {
                        tma_load_2d_pair(sa, &tmA, k0, m0, bar);
                    }
                    if (B_MN) {
#pragma unroll
                        for (int c = 0; c < (BN / 2) / 64; ++c) tma_load_2d_pair(sb + c * (BK * 128), &tmB, nb0 + c * 64, k0, bar);
                    } else {
                        tma_load_2d_pair(sb, &tmB, k0, nb0, bar);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer (first CTA only)
        if (lane == 0 && first) {
            const uint32_t idesc = make_idesc_f16(g.ab_format, A_MN ? 1 : 0, B_MN ? 1 : 0, 2 * BM, BN);
            uint32_t it = 0, tl = 0;
            for (int tile = pair; tile < total_tiles && !*abort_flag; tile += n_pairs, ++tl) {
                const int split = tile / tiles_mn;
                const int kb0 = split * g.kb_per_split, kb1 = min(kb_total, kb0 + g.kb_per_split);
                const uint32_t acc = tl & 1, acc_ph = (tl >> 1) & 1;
                if (!mbar_wait_bounded(tempty_bar + acc, acc_ph ^ 1)) { report(status, WAIT_TMEM_EMPTY, tile); *abort_flag = 1; break; }
                fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait_bounded(full_bar + s, ph)) { report(status, WAIT_FULL, s); *abort_flag = 1; break; }
                    fence_after_sync();
                    const uint32_t sa = smem_u32(smem + s * L::STAGE_BYTES);
                    const uint32_t sb = sa + L::A_BYTES;
#pragma unroll
                    for (int j = 0; j < BK / UMMA_K; ++j) {
                        const uint64_t da = A_MN ? make_smem_desc(sa + j * (UMMA_K * 128), BK * 128, 1024)
                                                 : make_smem_desc(sa + j * (UMMA_K * 2), 16, 1024);
                        const uint64_t db = B_MN ? make_smem_desc(sb + j * (UMMA_K * 128), BK * 128, 1024)
                                                 : make_smem_desc(sb + j * (UMMA_K * 2), 16, 1024);
                        if constexpr (ES == 2) mma_f16_ss_pair(d_tmem, da, db, idesc, (kb > kb0 || j > 0) ? 1u : 0u);
                        else mma_f8_ss_pair(d_tmem, da, db, idesc, (kb > kb0 || j > 0) ? 1u : 0u);
                    }
                    const uint32_t eb = smem_u32(empty_bar + s);
                    mma_commit_pair(eb);                       // this CTA's stage is reusable ...
                    mma_commit_pair(map_to_cta(eb, 1));        // ... and the partner's
                }
                const uint32_t tb = smem_u32(tfull_bar + acc);
                mma_commit_pair(tb);
                mma_commit_pair(map_to_cta(tb, 1));
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue (both CTAs: own 128 rows)
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;
        const int issuer = 64 + half * 128;
        const uint32_t tempty_first = map_to_cta(smem_u32(tempty_bar), 0);
        uint32_t tl = 0, oc = 0;
        for (int tile = pair; tile < total_tiles && !*abort_flag; tile += n_pairs, ++tl) {
            const int split = tile / tiles_mn;
            int tm, tn;
            tile_coords(tile - split * tiles_mn, tiles_m, tiles_n, tm, tn);
            const int m0 = tm * (2 * BM) + (int)rank * BM, n0 = tn * BN;
            const int row = m0 + quarter * 32 + lane;
            const uint32_t acc = tl & 1, acc_ph = (tl >> 1) & 1;
            bool ok = true;
            if (lane == 0) ok = mbar_wait_bounded(tfull_bar + acc, acc_ph);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) { if (lane == 0) { report(status, WAIT_TMEM_FULL, tile); *abort_flag = 1; } break; }
            fence_after_sync();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
#pragma unroll 1
            for (int c = half * (BN / 64); c < (half + 1) * (BN / 64); ++c) {
                uint32_t r[32];
                tmem_ld_32x32(taddr + c * 32, r);
                tmem_ld_wait();
                if (g.alpha != nullptr) {
#pragma unroll
                    for (int q = 0; q < 32; ++q) r[q] = __float_as_uint(__uint_as_float(r[q]) * alpha);
                }
                if (g.out_f32) {
                    // split-K partial sums / fp32 results: straight from registers, one 128-byte run per row
                    const int col0 = n0 + c * 32;
                    if (row < g.M && col0 < g.N) {
                        float* dst = reinterpret_cast<float*>(Dptr) + ((size_t)split * g.M + row) * g.ldd + col0;
                        if (col0 + 32 <= g.N) {
#pragma unroll
                            for (int q = 0; q < 8; ++q)
                                reinterpret_cast<uint4*>(dst)[q] = make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
                        } else {
#pragma unroll
                            for (int q = 0; q < 32; ++q)
                                if (col0 + q < g.N) dst[q] = __uint_as_float(r[q]);
                        }
                    }
                    continue;
                }
                uint8_t* stage_buf = smem + L::OUT_OFFSET + (half * 2 + (oc & 1)) * L::OUT_BYTES;
                if (oc >= 2 && (int)threadIdx.x == issuer) tma_store_wait_read<1>();
                ++oc;
                named_barrier(1 + half, 128);
                const int r_in_tile = quarter * 32 + lane;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint32_t w[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float lo = __uint_as_float(r[8 * q + 2 * e]), hi = __uint_as_float(r[8 * q + 2 * e + 1]);
                        if (g.out_bf16) { __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi); w[e] = *reinterpret_cast<uint32_t*>(&v); }
                        else { __half2 v = __floats2half2_rn(lo, hi); w[e] = *reinterpret_cast<uint32_t*>(&v); }
                    }
                    const int chunk = q ^ ((r_in_tile >> 1) & 3);
                    *reinterpret_cast<uint4*>(stage_buf + r_in_tile * 64 + chunk * 16) = make_uint4(w[0], w[1], w[2], w[3]);
                }
                fence_async_smem();
                named_barrier(1 + half, 128);
                if ((int)threadIdx.x == issuer) {
                    tma_store_2d(&tmD, stage_buf, n0 + c * 32, m0);
                    tma_store_commit();
                }
                if (g.stats != nullptr) {
                    const int cp = lane & 15, hi = lane >> 4;
                    float s1a = 0.f, s1b = 0.f, s2a = 0.f, s2b = 0.f;
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int rr = quarter * 32 + hi * 16 + ((i + hi) & 15);
                        const int chunk = (cp >> 2) ^ ((rr >> 1) & 3);
                        const uint32_t w = *reinterpret_cast<const uint32_t*>(stage_buf + rr * 64 + chunk * 16 + (cp & 3) * 4);
                        float lo, up;
                        if (g.out_bf16) { lo = __uint_as_float(w << 16); up = __uint_as_float(w & 0xffff0000u); }
                        else { const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w)); lo = f.x; up = f.y; }
                        s1a += lo; s1b += up; s2a = fmaf(lo, lo, s2a); s2b = fmaf(up, up, s2b);
                    }
                    s1a += __shfl_xor_sync(0xffffffffu, s1a, 16); s1b += __shfl_xor_sync(0xffffffffu, s1b, 16);
                    s2a += __shfl_xor_sync(0xffffffffu, s2a, 16); s2b += __shfl_xor_sync(0xffffffffu, s2b, 16);
                    const int col = n0 + c * 32 + cp * 2;
                    if (hi == 0 && col < g.N) {
                        float* dst = g.stats + ((size_t)((m0 / BM) * 4 + quarter) * 2) * g.N + col;
                        *reinterpret_cast<float2*>(dst) = make_float2(s1a, s1b);
                        *reinterpret_cast<float2*>(dst + g.N) = make_float2(s2a, s2b);
                    }
                }
            }
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tempty_first + acc * 8);      // the MMA thread lives in the first CTA
        }
        if ((int)threadIdx.x == issuer) tma_store_wait_all<0>();
    }

    // -------------------------------------------------------------------- teardown
    if (*abort_flag) {
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    fence_before_sync();
    __syncthreads();
    cluster_sync_all();                                      // the partner is done with this CTA's shared memory and TMEM
    fence_after_sync();
    if (warp == 1) tmem_dealloc_pair(tmem_base, 2 * BN);
}

// out[m, n] = sum_s partial[s, m, n]   (fixed order), cast to OUT
template <typename OUT>
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, OUT* __restrict__ out, long long mn, int splits,
                                     float beta, const OUT* __restrict__ prev) {
    const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= mn) return;
    float4 acc = *reinterpret_cast<const float4*>(partial + i);
    for (int s = 1; s < splits; ++s) {
        const float4 p = *reinterpret_cast<const float4*>(partial + (long long)s * mn + i);
        acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
    }
    float v[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        if (i + q < mn) {
            float r = v[q];
            if (prev != nullptr) r += beta * (float)prev[i + q];
            out[i + q] = (OUT)r;
        }
    }
}

// ---- host side ---------------------------------------------------------------------
template <int BN, int STAGES, bool A_MN, bool B_MN, int ES = 2>
void launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td, void* d, const GemmArgs& g,
            KernelStatus* st, int grid, cudaStream_t stream) {
    using L = SmemLayout<BN, STAGES>;
    auto kern = gemm_kernel<BN, STAGES, A_MN, B_MN, ES>;
    static bool configured = false;
    if (!configured) {
        C10_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
        configured = true;
    }
    kern<<<grid, kThreads, L::TOTAL, stream>>>(ta, tb, td, d, g, st);
}

template <bool A_MN, bool B_MN, int ES = 2>
void launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td, void* d, const GemmArgs& g, KernelStatus* st,
                 int grid, cudaStream_t stream) {
    auto kern = gemm_pair_kernel<A_MN, B_MN, ES>;
    static bool configured = false;
    if (!configured) {
        C10_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PairSmem::TOTAL));
        configured = true;
    }
    kern<<<grid, kThreads, PairSmem::TOTAL, stream>>>(ta, tb, td, d, g, st);
}

// 0: never use CTA pairs; 1: use them where they measured faster (M, N >= 256 and >= 16 k-blocks); 2: wherever possible
int& pair_mode() {
    static int mode = []() {
        const char* e = std::getenv("SJB200_GEMM_PAIR");
        return e != nullptr ? std::atoi(e) : 1;
    }();
    return mode;
}

}  // namespace

// D = A (.) B with fp32 accumulation.
//   a_mn == false: `a` is [M, K] (K contiguous);  a_mn == true: `a` is [K, M] (M contiguous)
//   b_mn == false: `b` is [N, K] (K contiguous);  b_mn == true: `b` is [K, N] (N contiguous)
//   out_f32: result dtype fp32 instead of the input dtype;  split_k: 0 = choose, else forced
static at::Tensor gemm_16bit_impl(const at::Tensor& a, const at::Tensor& b, bool a_mn, bool b_mn, bool out_f32, int64_t split_k,
                                  at::Tensor* stats) {
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
    at::Tensor out = at::empty({M, N}, out_f32 ? opts.dtype(at::kFloat) : opts);
    at::Tensor scratch;
    void* dptr = out.data_ptr();
    if (splits > 1) {
        scratch = at::empty({splits, M, N}, opts.dtype(at::kFloat));
        dptr = scratch.data_ptr();
    }
    // 16-bit results leave through TMA (box 128 x 32, 64-byte swizzle); fp32 results are stored directly
    const CUtensorMap td = g.out_f32 ? ta : make_map(out.data_ptr(), M, N, N, BM, bf16, 32);
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

// The same product plus partial[blk][0 | 1][n] = sum | sum of squares of D[32 * blk .. 32 * blk + 31][n] (rows past M
// count as zero), taken from the rounded 16-bit values inside the epilogue: a following batch norm needs no pass over D.
std::tuple<at::Tensor, at::Tensor> gemm_16bit_stats(const at::Tensor& a, const at::Tensor& b, bool a_mn, bool b_mn) {
    at::Tensor stats;
    at::Tensor out = gemm_16bit_impl(a, b, a_mn, b_mn, false, 1, &stats);
    return {out, stats};
}

// D[M, N] (bf16) = alpha * A[M, K] (.) B[N, K]^T with fp8 operands (both e4m3 or both e5m2, K contiguous) and fp32
// accumulation on the tensor cores.  `alpha`: optional fp32 device scalar (the product of the two
// de-quantisation scales), multiplied in the epilogue so that no host synchronisation is needed.
at::Tensor gemm_fp8(const at::Tensor& a, const at::Tensor& b, const c10::optional<at::Tensor>& alpha, bool out_f32,
                    int64_t split_k) {
    TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.dim() == 2 && b.dim() == 2, "gemm_fp8: 2-D CUDA operands required");
    const bool e4m3 = a.scalar_type() == at::kFloat8_e4m3fn, e5m2 = a.scalar_type() == at::kFloat8_e5m2;
    TORCH_CHECK((e4m3 || e5m2) && a.scalar_type() == b.scalar_type(), "gemm_fp8: both operands must be float8_e4m3fn or both float8_e5m2");
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
    g.ab_format = e4m3 ? 0 : 1;
    g.out_bf16 = 1;
    g.alpha = nullptr;
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
    const CUtensorMap td = g.out_f32 ? ta : make_map(out.data_ptr(), M, N, N, BM, true, 32);
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
    m.def("gemm_fp8(Tensor a, Tensor b, Tensor? alpha, bool out_f32, int split_k) -> Tensor");
    m.def("gemm_status(Tensor like) -> int[]");
    m.def("gemm_set_pair_mode(int mode) -> int");
}
TORCH_LIBRARY_IMPL(sjb200, CompositeExplicitAutograd, m) {
    m.impl("gemm_set_pair_mode", &sjb200::gemm_set_pair_mode);
}
TORCH_LIBRARY_IMPL(sjb200, CUDA, m) {
    m.impl("gemm_16bit", &sjb200::gemm_16bit);
    m.impl("gemm_16bit_stats", &sjb200::gemm_16bit_stats);
    m.impl("gemm_fp8", &sjb200::gemm_fp8);
    m.impl("gemm_status", &sjb200::gemm_status);
}
