// Tensor-parallel spiking linear layers with the collective inside the GEMM.
//
//   spike_gemm:  D[M, N] = S[M, K] . W[N, K]^T      S = spikes, stored as 1 bit per element
//
// * The A operand never exists as 16-bit data in global memory.  Four "expander" warps read the packed bits of
//   their 128 rows with plain loads, turn every pair of bits into two bf16 values with integer arithmetic and
//   write the 128-byte-swizzled K-major tile that tcgen05.mma expects; the weights arrive by TMA.
//   The rows of one 128-row tile may live on ANOTHER GPU: the tile's base pointer is taken from a table of
//   peer-mapped symmetric buffers.  That is the all-gather of a column-parallel layer, moved into the GEMM's
//   operand fetch with a payload of 1 bit per activation (each CTA fetches the rows it needs itself; no TMA
//   and no multicast touch peer memory).
// * Epilogue 0 stores bf16 rows locally.  Epilogue 1 is the reduce-scatter of a row-parallel layer: every
//   finished 128 x 32 chunk of the partial product is stored straight into the staging buffer of the rank
//   that owns those rows (peer stores), slot [this rank], while the tensor cores work on the next tile.
//   After a barrier the owner adds the slots in rank order (`tp_reduce_residual`), so the sum is deterministic.
// * Rows are ordered [t][token]; tokens are split evenly over the ranks, so rank o owns
//   rows {t * tokens + o * tokens_per_rank + i}.  tokens_per_rank must be a multiple of 128 (one tile never
//   straddles two owners).
// * `tp_barrier` is the bounded flag barrier shared with the all-reduce: on expiry it records the peer in a
//   status word and returns.  Every mbarrier wait in the GEMM is bounded as well.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_bf16.h>
#include <torch/library.h>

#include "comm_common.cuh"
#include "tc_common.cuh"
#include "tma_host.cuh"

namespace sjb200 {
namespace {

using namespace tc;

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kThreads = 448;       // warps: 0 TMA(B), 1 MMA, 2-5 epilogue, 6-9 A expanders (even k-blocks), 10-13 (odd)
constexpr int kMaxRanks = 8;

template <int BN, int STAGES>
struct Smem {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
    static constexpr int OUT_OFFSET = BAR_OFFSET + 1024;              // epilogue staging: 4 warps x [32 rows][64 cols] bf16
    static constexpr int TOTAL = OUT_OFFSET + 4 * 4096 + 1024;        // + slack for 1024 B alignment
};

struct SpikeGemmArgs {
    int M, N, K;                 // K = number of spike columns actually multiplied (weights are zero-filled beyond)
    int ldd;                     // leading dimension of a local D (elements)
    long long a_pitch;           // bytes per packed row (multiple of 32)
    int rows_per_t;              // tokens in total (rows of one time step)
    int rows_per_src;            // tokens per rank
    int rank, world;
    const uint8_t* a_src[kMaxRanks];   // packed spikes of every rank, rows [t][local token]
    __nv_bfloat16* d_dst[kMaxRanks];   // EPI 1: staging buffer of every rank, [world][T * rows_per_src][N]
    __nv_bfloat16* d_local;            // EPI 0
    long long slot_elems;              // EPI 1: elements of one staging slot (T * rows_per_src * N)
};

// row block [m0, m0 + 128) -> (rank that holds / owns it, row inside that rank's buffer).  `sharded == false`:
// the whole matrix is local.
__device__ __forceinline__ void locate(const SpikeGemmArgs& g, bool sharded, int m0, int& src, long long& local_row) {
    if (!sharded) { src = 0; local_row = m0; return; }
    const int t = m0 / g.rows_per_t, tok = m0 - t * g.rows_per_t;
    src = tok / g.rows_per_src;
    local_row = (long long)t * g.rows_per_src + (tok - src * g.rows_per_src);
}

template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(kThreads, 1)
spike_gemm_kernel(const __grid_constant__ CUtensorMap tmB, const SpikeGemmArgs g, KernelStatus* __restrict__ status) {
    using L = Smem<BN, STAGES>;
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
    const int total_tiles = tiles_m * tiles_n;
    const int kb_total = (g.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        // full: one arrival from the TMA thread (with the byte count) + one from each of the four expander warps
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar + s, 5); mbar_init(empty_bar + s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar + a, 1); mbar_init(tempty_bar + a, 4); }
        *abort_flag = 0;
        mbar_init_fence();
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
        // ------------------------------------------------------------ TMA producer (weights)
        if (lane == 0) {
            uint32_t it = 0;
            for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x) {
                const int n0 = (tile % tiles_n) * BN;
                for (int kb = 0; kb < kb_total; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait_bounded(empty_bar + s, ((it / STAGES) & 1) ^ 1)) { report(status, WAIT_EMPTY, s); *abort_flag = 1; break; }
                    mbar_expect_tx(full_bar + s, L::B_BYTES);
                    tma_load_2d(smem + s * L::STAGE_BYTES + L::A_BYTES, &tmB, kb * BK, n0, full_bar + s);
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            const uint32_t idesc = make_idesc_f16(1, 0, 0, BM, BN);
            uint32_t it = 0, tl = 0;
            for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x, ++tl) {
                const uint32_t acc = tl & 1, acc_ph = (tl >> 1) & 1;
                if (!mbar_wait_bounded(tempty_bar + acc, acc_ph ^ 1)) { report(status, WAIT_TMEM_EMPTY, tile); *abort_flag = 1; break; }
                fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < kb_total; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait_bounded(full_bar + s, (it / STAGES) & 1)) { report(status, WAIT_FULL, s); *abort_flag = 1; break; }
                    fence_after_sync();
                    const uint32_t sa = smem_u32(smem + s * L::STAGE_BYTES);
                    const uint32_t sb = sa + L::A_BYTES;
#pragma unroll
                    for (int j = 0; j < BK / UMMA_K; ++j)
                        mma_f16_ss(d_tmem, make_smem_desc(sa + j * (UMMA_K * 2), 16, 1024), make_smem_desc(sb + j * (UMMA_K * 2), 16, 1024),
                                   idesc, (kb > 0 || j > 0) ? 1u : 0u);
                    mma_commit(empty_bar + s);
                }
                mma_commit(tfull_bar + acc);
            }
        }
    } else if (warp >= 6) {
        // -------------------------------------------------------------- A expanders: bits -> swizzled bf16 tile
        // Two groups of four warps take the even and the odd k-blocks.  Inside a group each warp owns 32 rows and
        // reports to the stage barrier on its own (no block-wide rendezvous).  A thread
        // reads its row 32 bytes (= 4 k-blocks) at a time and keeps two such groups in flight ahead of the one
        // it expands, which covers the latency of a peer load over NVLink.
        const int r = (threadIdx.x - 192) & 127;         // row of the tile owned by this thread
        const int parity = (threadIdx.x - 192) >> 7;     // which k-blocks this thread expands
        const uint32_t swz = (uint32_t)(r & 7);
        const int groups = (kb_total + 3) >> 2;
        uint32_t it = 0;
        bool dead = false;
        for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag && !dead; tile += gridDim.x) {
            const int m0 = (tile / tiles_n) * BM;
            int src; long long local_row;
            locate(g, g.world > 1, m0, src, local_row);
            const bool live = m0 + r < g.M;
            const uint4* rowp = reinterpret_cast<const uint4*>(g.a_src[src] + (local_row + r) * g.a_pitch);
            const uint4 zero4 = make_uint4(0, 0, 0, 0);
            uint4 c0 = zero4, c1 = zero4, n0 = zero4, n1 = zero4, f0 = zero4, f1 = zero4;   // current, next, after next
            if (live) {
                c0 = __ldcg(rowp); c1 = __ldcg(rowp + 1);
                if (groups > 1) { n0 = __ldcg(rowp + 2); n1 = __ldcg(rowp + 3); }
            }
            int kb = 0;
            for (int grp = 0; grp < groups && !dead; ++grp) {
                if (live && grp + 2 < groups) { f0 = __ldcg(rowp + 2 * (grp + 2)); f1 = __ldcg(rowp + 2 * (grp + 2) + 1); }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (kb >= kb_total) break;
                    if ((j & 1) != parity) { ++kb; ++it; continue; }
                    const int s = it % STAGES;
                    bool ok = true;
                    if (lane == 0) ok = mbar_wait_bounded(empty_bar + s, ((it / STAGES) & 1) ^ 1);
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) { if (lane == 0) { report(status, WAIT_EMPTY, 100 + s); *abort_flag = 1; } dead = true; break; }
                    const uint4 c4 = (j & 2) ? c1 : c0;
                    const uint32_t w0 = (j & 1) ? c4.z : c4.x, w1 = (j & 1) ? c4.w : c4.y;
                    uint8_t* arow = smem + s * L::STAGE_BYTES + r * 128;
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        const uint32_t byte = ((c < 4 ? w0 : w1) >> (8 * (c & 3))) & 0xFFu;
                        uint32_t w[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const uint32_t x = (byte >> (2 * e)) & 3u;            // two spikes
                            w[e] = ((x * 0x8001u) & 0x00010001u) * 0x3F80u;        // -> two bf16 (1.0 = 0x3F80)
                        }
                        *reinterpret_cast<uint4*>(arow + ((c ^ swz) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                    fence_async_smem();                  // generic-proxy writes -> visible to the tensor core's async proxy
                    __syncwarp();
                    if (lane == 0) mbar_arrive(full_bar + s);
                    ++kb; ++it;
                }
                c0 = n0; c1 = n1; n0 = f0; n1 = f1;
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        const int quarter = warp & 3;
        uint32_t tl = 0;
        for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x, ++tl) {
            const int m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * BN;
            const uint32_t acc = tl & 1, acc_ph = (tl >> 1) & 1;
            bool ok = true;
            if (lane == 0) ok = mbar_wait_bounded(tfull_bar + acc, acc_ph);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) { if (lane == 0) { report(status, WAIT_TMEM_FULL, tile); *abort_flag = 1; } break; }
            fence_after_sync();
            const int row = m0 + quarter * 32 + lane;
            // rows of one tile share their owner (row blocks of a source rank are multiples of BM)
            __nv_bfloat16* dtile;                        // row `m0 + quarter * 32` of the destination
            if (EPI == 0) {
                dtile = g.d_local + (size_t)(m0 + quarter * 32) * g.ldd;
            } else {
                int owner; long long local_row;
                locate(g, true, m0, owner, local_row);
                dtile = g.d_dst[owner] + (size_t)g.rank * g.slot_elems + (size_t)(local_row + quarter * 32) * g.N;
            }
            const size_t dld = EPI == 0 ? (size_t)g.ldd : (size_t)g.N;
            __nv_bfloat16* drow = dtile + (size_t)lane * dld;
            uint8_t* stg = smem + L::OUT_OFFSET + quarter * 4096;      // this warp's [32][64] bf16, 16-byte chunks XOR (row & 7)
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t rr[32];
                tmem_ld_32x32(taddr + c * 32, rr);
                tmem_ld_wait();
                const int col0 = n0 + c * 32;
                uint32_t w[16];
#pragma unroll
                for (int q = 0; q < 16; ++q) {
                    __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(rr[2 * q]), __uint_as_float(rr[2 * q + 1]));
                    w[q] = *reinterpret_cast<uint32_t*>(&v);
                }
                const int pair0 = n0 + (c & ~1) * 32;    // first column of the 64-column pair this chunk belongs to
                if (pair0 + 64 <= g.N) {
                    // Stage two 32-column chunks, then leave as 128-byte row segments: eight lanes per row, four rows per
                    // store instruction.  A lane-per-row store would put 32 separate 16-byte pieces on the wire, which is
                    // what made the peer push slow over NVLink.
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        *reinterpret_cast<uint4*>(stg + lane * 128 + ((((c & 1) * 4 + q) ^ (lane & 7)) << 4)) =
                            make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
                    if (c & 1) {
                        __syncwarp();
                        const int ch = lane & 7;
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int r = i * 4 + (lane >> 3);
                            const uint4 v = *reinterpret_cast<const uint4*>(stg + r * 128 + ((ch ^ (r & 7)) << 4));
                            if (m0 + quarter * 32 + r < g.M)
                                *reinterpret_cast<uint4*>(dtile + (size_t)r * dld + pair0 + ch * 8) = v;
                        }
                        __syncwarp();
                    }
                } else if (row < g.M && col0 < g.N) {
                    if (col0 + 32 <= g.N) {
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            reinterpret_cast<uint4*>(drow + col0)[q] = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
                    } else {
#pragma unroll
                        for (int q = 0; q < 16; ++q)
                            if (col0 + 2 * q < g.N) *reinterpret_cast<uint32_t*>(drow + col0 + 2 * q) = w[q];
                    }
                }
            }
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar + acc);
        }
        if (EPI == 1) __threadfence_system();            // peer stores are performed before the kernel is seen as finished
    }

    if (*abort_flag) {
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    if (warp == 1) tmem_dealloc(tmem_base, 2 * BN);
}

// ---------------------------------------------------------------------------------------------------------------
// LIF over T on a [T, rows, C] bf16 tensor, spikes written as bits: out[(t * rows + row) * pitch + c / 8].
// hard reset to 0, decay_input: h = v + (x - v) / tau.   One thread = 8 consecutive columns of one row.
__global__ void __launch_bounds__(256)
lif_pack_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ out, int T, long long rows, int C, long long pitch,
                float inv_tau, float v_th) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int groups = C >> 3;
    if (i >= rows * groups) return;
    const long long row = i / groups;
    const int cg = (int)(i - row * groups);
    float v[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) v[q] = 0.f;
    for (int t = 0; t < T; ++t) {
        const uint4 raw = *reinterpret_cast<const uint4*>(x + ((size_t)t * rows + row) * C + cg * 8);
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
        uint32_t bits = 0;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float2 f = __bfloat1622float2(p[q]);
            const float in[2] = {f.x, f.y};
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int k = 2 * q + e;
                const float h = __fadd_rn(v[k], __fmul_rn(__fsub_rn(in[e], v[k]), inv_tau));
                const bool s = h >= v_th;
                bits |= (s ? 1u : 0u) << k;
                v[k] = s ? 0.f : h;
            }
        }
        out[((size_t)t * rows + row) * pitch + cg] = (uint8_t)bits;
    }
}

// RMSNorm over C, then the same LIF, then bit-pack.  h: [T, rows, C] (fp32 or bf16); one block per row;
// blockDim.x * 8 == C.
struct PackDst {
    uint8_t* p[comm::kMaxWorld];   // where this rank's packed rows go: one buffer per rank of the group (its own included)
    int n;
};

template <typename HT>
__global__ void __launch_bounds__(512)
rmsnorm_lif_pack_kernel(const HT* __restrict__ h, const float* __restrict__ weight, PackDst dst, int T, long long rows,
                        int C, long long pitch, float eps, float inv_tau, float v_th) {
    __shared__ float red[16];
    const long long row = blockIdx.x;
    const int c0 = threadIdx.x * 8;
    float w[8], v[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) { w[q] = weight[c0 + q]; v[q] = 0.f; }
    for (int t = 0; t < T; ++t) {
        float x[8];
        const HT* p = h + ((size_t)t * rows + row) * C + c0;
        if constexpr (sizeof(HT) == 4) {
            const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
            x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
        } else {
            const uint4 raw = *reinterpret_cast<const uint4*>(p);
            const __nv_bfloat162* pp = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int q = 0; q < 4; ++q) { const float2 f = __bfloat1622float2(pp[q]); x[2 * q] = f.x; x[2 * q + 1] = f.y; }
        }
        float ss = 0.f;
#pragma unroll
        for (int q = 0; q < 8; ++q) ss += x[q] * x[q];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        __syncthreads();                                  // `red` of the previous step has been read by everyone
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
        __syncthreads();
        float tot = 0.f;
        for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += red[i];
        const float rinv = rsqrtf(tot / (float)C + eps);
        uint32_t bits = 0;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const float in = x[q] * rinv * w[q];
            const float hh = __fadd_rn(v[q], __fmul_rn(__fsub_rn(in, v[q]), inv_tau));
            const bool s = hh >= v_th;
            bits |= (s ? 1u : 0u) << q;
            v[q] = s ? 0.f : hh;
        }
        // sixteen lanes' bytes travel as one 16-byte store per destination (a peer store of single bytes would
        // put one NVLink packet on the wire per byte)
        const uint32_t full = 0xffffffffu;
        const uint32_t w32 = bits | (__shfl_down_sync(full, bits, 1) << 8) | (__shfl_down_sync(full, bits, 2) << 16) |
                             (__shfl_down_sync(full, bits, 3) << 24);
        uint4 q;
        q.x = w32; q.y = __shfl_down_sync(full, w32, 4); q.z = __shfl_down_sync(full, w32, 8); q.w = __shfl_down_sync(full, w32, 12);
        if ((threadIdx.x & 15) == 0) {
            const size_t off = ((size_t)t * rows + row) * pitch + threadIdx.x;
            for (int d = 0; d < dst.n; ++d) *reinterpret_cast<uint4*>(dst.p[d] + off) = q;
        }
    }
}

// h[i] += sum over slots s (rank order) of stage[s][i]
template <typename HT>
__global__ void __launch_bounds__(256)
reduce_residual_kernel(HT* __restrict__ h, const __nv_bfloat16* __restrict__ stage, long long n, long long slot_elems, int world) {
    const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (i >= n) return;
    float acc[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) acc[q] = 0.f;
    for (int s = 0; s < world; ++s) {
        const uint4 raw = *reinterpret_cast<const uint4*>(stage + (size_t)s * slot_elems + i);
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int q = 0; q < 4; ++q) { const float2 f = __bfloat1622float2(p[q]); acc[2 * q] += f.x; acc[2 * q + 1] += f.y; }
    }
    if constexpr (sizeof(HT) == 4) {
        float4* hp = reinterpret_cast<float4*>(h + i);
        float4 a = hp[0], b = hp[1];
        a.x += acc[0]; a.y += acc[1]; a.z += acc[2]; a.w += acc[3]; b.x += acc[4]; b.y += acc[5]; b.z += acc[6]; b.w += acc[7];
        hp[0] = a; hp[1] = b;
    } else {
        uint4 raw = *reinterpret_cast<uint4*>(h + i);
        __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float2 f = __bfloat1622float2(p[q]);
            p[q] = __floats2bfloat162_rn(f.x + acc[2 * q], f.y + acc[2 * q + 1]);
        }
        *reinterpret_cast<uint4*>(h + i) = raw;
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Pieces of the training path: an all-gather as peer stores of whole chunks, and a reduce-scatter as peer loads.
struct ChunkPeers {
    uint8_t* p[comm::kMaxWorld];
    int n;
};

// Chunk c (chunk_bytes, contiguous in src) is stored at dst + c * dst_stride for every destination: with
// chunks = T this lays one rank's [T][n][row] block into everybody's [T][world * n][row] buffer.
__global__ void __launch_bounds__(256)
push_chunks_kernel(const uint4* __restrict__ src, ChunkPeers dst, long long vec_per_chunk, long long dst_stride_vec, long long total_vec) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total_vec; i += (long long)gridDim.x * blockDim.x) {
        const long long c = i / vec_per_chunk, r = i - c * vec_per_chunk;
        const uint4 v = src[i];
        for (int d = 0; d < dst.n; ++d) reinterpret_cast<uint4*>(dst.p[d])[c * dst_stride_vec + r] = v;
    }
    __threadfence_system();
}

// out[c][r] = sum over sources j (rank order, fp32) of src_j[c * src_stride + r]: this rank's chunk of every peer's
// partial result, read in place over NVLink.
template <typename OT>
__global__ void __launch_bounds__(256)
reduce_chunks_kernel(ChunkPeers src, OT* __restrict__ out, long long vec_per_chunk, long long src_stride_vec, long long total_vec) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total_vec; i += (long long)gridDim.x * blockDim.x) {
        const long long c = i / vec_per_chunk, r = i - c * vec_per_chunk;
        uint4 v[comm::kMaxWorld];
#pragma unroll
        for (int j = 0; j < comm::kMaxWorld; ++j)
            if (j < src.n) v[j] = reinterpret_cast<const uint4*>(src.p[j])[c * src_stride_vec + r];
        float acc[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[q] = 0.f;
#pragma unroll
        for (int j = 0; j < comm::kMaxWorld; ++j)
            if (j < src.n) {
                const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v[j]);
#pragma unroll
                for (int q = 0; q < 4; ++q) { const float2 f = __bfloat1622float2(p[q]); acc[2 * q] += f.x; acc[2 * q + 1] += f.y; }
            }
        if constexpr (sizeof(OT) == 4) {
            float4* o = reinterpret_cast<float4*>(out + i * 8);
            o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
            o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
        } else {
            uint4 w;
            __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
            for (int q = 0; q < 4; ++q) p[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
            reinterpret_cast<uint4*>(out)[i] = w;
        }
    }
}

__global__ void tp_barrier_kernel(comm::PeerPtrs pp, int rank, int world, uint32_t epoch, comm::CommStatus* status, long long timeout_ns) {
    __threadfence_system();
    comm::block_barrier(pp, rank, world, 1, epoch, 1, status, timeout_ns);
}

template <int BN, int STAGES, int EPI>
void launch_spike_gemm(const CUtensorMap& tb, const SpikeGemmArgs& g, KernelStatus* st, int grid, cudaStream_t stream) {
    using L = Smem<BN, STAGES>;
    auto kern = spike_gemm_kernel<BN, STAGES, EPI>;
    static bool configured = false;
    if (!configured) {
        C10_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
        configured = true;
    }
    kern<<<grid, kThreads, L::TOTAL, stream>>>(tb, g, st);
}

}  // namespace

// a_ptrs: device addresses of every rank's packed spikes (one entry = plain local operand); rows are [t][token].
// push_ptrs: empty -> result returned as a local bf16 [M, N]; else the staging buffers of every rank and the
// partial product is scattered to the owners (nothing is returned: an empty tensor).
at::Tensor spike_gemm(std::vector<int64_t> a_ptrs, int64_t a_pitch, int64_t M, int64_t K, const at::Tensor& w,
                      int64_t rows_per_t, int64_t rows_per_src, int64_t rank, std::vector<int64_t> push_ptrs, int64_t slot_elems) {
    TORCH_CHECK(w.is_cuda() && w.dim() == 2 && w.scalar_type() == at::kBFloat16 && w.stride(1) == 1, "spike_gemm: bf16 weight [N, K] required");
    const int world = (int)a_ptrs.size();
    TORCH_CHECK(world >= 1 && world <= kMaxRanks, "spike_gemm: 1..8 sources");
    TORCH_CHECK(a_pitch % 32 == 0 && a_pitch * 8 >= K, "spike_gemm: packed rows must be padded to a multiple of 32 bytes");
    TORCH_CHECK(K <= w.size(1), "spike_gemm: more spike columns than weight columns");
    const bool push = !push_ptrs.empty();
    TORCH_CHECK(!push || (int)push_ptrs.size() <= kMaxRanks, "spike_gemm: too many destinations");
    if (world > 1 || push) {
        TORCH_CHECK(rows_per_src % BM == 0 && rows_per_t % rows_per_src == 0 && M % rows_per_t == 0,
                    "spike_gemm: tokens per rank must be a multiple of 128 and divide the rows of a step");
    }
    const int64_t N = w.size(0);
    TORCH_CHECK(N % 8 == 0, "spike_gemm: N must be a multiple of 8");
    const c10::cuda::CUDAGuard guard(w.device());
    C10_CUDA_CHECK(cudaFree(nullptr));

    SpikeGemmArgs g{};
    g.M = (int)M; g.N = (int)N; g.K = (int)K; g.ldd = (int)N;
    g.a_pitch = a_pitch; g.rows_per_t = (int)rows_per_t; g.rows_per_src = (int)rows_per_src;
    g.rank = (int)rank; g.world = world; g.slot_elems = slot_elems;
    for (int j = 0; j < world; ++j) {
        TORCH_CHECK(a_ptrs[j] % 16 == 0, "spike_gemm: packed spikes must be 16-byte aligned");
        g.a_src[j] = reinterpret_cast<const uint8_t*>(a_ptrs[j]);
    }
    at::Tensor out;
    if (push) {
        for (size_t j = 0; j < push_ptrs.size(); ++j) g.d_dst[j] = reinterpret_cast<__nv_bfloat16*>(push_ptrs[j]);
        out = at::empty({0}, w.options());
    } else {
        out = at::empty({M, N}, w.options());
        g.d_local = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
    }
    const int BN = N > 128 ? 256 : 128;
    const CUtensorMap tb = make_map(w.data_ptr(), N, w.size(1), w.stride(0), BN, true);
    const int tiles = (int)(((M + BM - 1) / BM) * ((N + BN - 1) / BN));
    const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    const int grid = std::min(tiles, sms);
    at::Tensor& st = status_word(w.device());
    KernelStatus* stp = reinterpret_cast<KernelStatus*>(st.data_ptr<int>());
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    if (BN == 256) { if (push) launch_spike_gemm<256, 4, 1>(tb, g, stp, grid, stream); else launch_spike_gemm<256, 4, 0>(tb, g, stp, grid, stream); }
    else { if (push) launch_spike_gemm<128, 6, 1>(tb, g, stp, grid, stream); else launch_spike_gemm<128, 6, 0>(tb, g, stp, grid, stream); }
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return out;
}

// x: [T, rows, C] bf16 -> bits written at out_ptr with `pitch` bytes per (t, row)
void lif_pack(const at::Tensor& x, int64_t out_ptr, int64_t pitch, double tau, double v_th) {
    TORCH_CHECK(x.is_cuda() && x.dim() == 3 && x.is_contiguous() && x.scalar_type() == at::kBFloat16, "lif_pack: contiguous bf16 [T, rows, C]");
    const int T = (int)x.size(0), C = (int)x.size(2);
    const long long rows = x.size(1);
    TORCH_CHECK(C % 8 == 0 && pitch * 8 >= C, "lif_pack: C must be a multiple of 8 and fit the pitch");
    const c10::cuda::CUDAGuard guard(x.device());
    const long long n = rows * (C / 8);
    lif_pack_kernel<<<(unsigned)((n + 255) / 256), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
        reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), reinterpret_cast<uint8_t*>(out_ptr), T, rows, C, pitch, (float)(1.0 / tau), (float)v_th);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// Packed spikes of LIF_T(RMSNorm(h)) are written to every pointer of `out_ptrs` (the same bytes to each): with the peers'
// gather buffers in the list the all-gather of the spikes happens as stores out of the producing kernel.
void rmsnorm_lif_pack(const at::Tensor& h, const at::Tensor& weight, std::vector<int64_t> out_ptrs, int64_t pitch, double eps, double tau, double v_th) {
    TORCH_CHECK(h.is_cuda() && h.dim() == 3 && h.is_contiguous(), "rmsnorm_lif_pack: contiguous [T, rows, C]");
    TORCH_CHECK(weight.scalar_type() == at::kFloat && weight.is_contiguous() && weight.numel() == h.size(2), "rmsnorm_lif_pack: fp32 weight [C]");
    const int T = (int)h.size(0), C = (int)h.size(2);
    const long long rows = h.size(1);
    TORCH_CHECK(C % 256 == 0 && C <= 4096 && pitch * 8 >= C, "rmsnorm_lif_pack: C must be a multiple of 256, at most 4096");
    const c10::cuda::CUDAGuard guard(h.device());
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    TORCH_CHECK(!out_ptrs.empty() && (int)out_ptrs.size() <= comm::kMaxWorld && pitch % 16 == 0, "rmsnorm_lif_pack: 1..16 destinations, pitch a multiple of 16");
    PackDst out{};
    out.n = (int)out_ptrs.size();
    for (int d = 0; d < out.n; ++d) {
        TORCH_CHECK(out_ptrs[d] % 16 == 0, "rmsnorm_lif_pack: destinations must be 16-byte aligned");
        out.p[d] = reinterpret_cast<uint8_t*>(out_ptrs[d]);
    }
    if (h.scalar_type() == at::kFloat)
        rmsnorm_lif_pack_kernel<float><<<(unsigned)rows, C / 8, 0, st>>>(h.data_ptr<float>(), weight.data_ptr<float>(), out, T, rows, C, pitch, (float)eps, (float)(1.0 / tau), (float)v_th);
    else if (h.scalar_type() == at::kBFloat16)
        rmsnorm_lif_pack_kernel<__nv_bfloat16><<<(unsigned)rows, C / 8, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(h.data_ptr()), weight.data_ptr<float>(), out, T, rows, C, pitch, (float)eps, (float)(1.0 / tau), (float)v_th);
    else TORCH_CHECK(false, "rmsnorm_lif_pack: fp32 or bf16 input");
    C10_CUDA_KERNEL_LAUNCH_CHECK();
}

void tp_reduce_residual(at::Tensor h, int64_t stage_ptr, int64_t slot_elems, int64_t world) {
    TORCH_CHECK(h.is_cuda() && h.is_contiguous() && h.numel() % 8 == 0 && h.numel() <= slot_elems, "tp_reduce_residual: bad residual tensor");
    const c10::cuda::CUDAGuard guard(h.device());
    const long long n = h.numel();
    const unsigned blocks = (unsigned)((n / 8 + 255) / 256);
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    const __nv_bfloat16* stage = reinterpret_cast<const __nv_bfloat16*>(stage_ptr);
    if (h.scalar_type() == at::kFloat) reduce_residual_kernel<float><<<blocks, 256, 0, st>>>(h.data_ptr<float>(), stage, n, slot_elems, (int)world);
    else if (h.scalar_type() == at::kBFloat16) reduce_residual_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(reinterpret_cast<__nv_bfloat16*>(h.data_ptr()), stage, n, slot_elems, (int)world);
    else TORCH_CHECK(false, "tp_reduce_residual: fp32 or bf16 residual");
    C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// src: contiguous, `chunks` pieces of equal size.  Piece c is written to dst_ptrs[j] + dst_offset_bytes + c * dst_stride_bytes
// on every rank j of the list (this rank's own buffer included).  All sizes are multiples of 16 bytes.
void tp_push_chunks(const at::Tensor& src, std::vector<int64_t> dst_ptrs, int64_t chunks, int64_t dst_stride_bytes, int64_t dst_offset_bytes) {
    TORCH_CHECK(src.is_cuda() && src.is_contiguous(), "tp_push_chunks: contiguous CUDA tensor required");
    const int64_t total = src.numel() * src.element_size();
    TORCH_CHECK(chunks >= 1 && total % chunks == 0, "tp_push_chunks: the tensor does not split into equal chunks");
    const int64_t chunk_bytes = total / chunks;
    TORCH_CHECK(chunk_bytes % 16 == 0 && dst_stride_bytes % 16 == 0 && dst_offset_bytes % 16 == 0 &&
                reinterpret_cast<uintptr_t>(src.data_ptr()) % 16 == 0, "tp_push_chunks: 16-byte granularity required");
    TORCH_CHECK(!dst_ptrs.empty() && (int)dst_ptrs.size() <= comm::kMaxWorld, "tp_push_chunks: 1..16 destinations");
    const c10::cuda::CUDAGuard guard(src.device());
    ChunkPeers dst{};
    dst.n = (int)dst_ptrs.size();
    for (int j = 0; j < dst.n; ++j) {
        TORCH_CHECK(dst_ptrs[j] % 16 == 0, "tp_push_chunks: destinations must be 16-byte aligned");
        dst.p[j] = reinterpret_cast<uint8_t*>(dst_ptrs[j] + dst_offset_bytes);
    }
    const long long total_vec = total / 16;
    const unsigned blocks = (unsigned)std::min<long long>((total_vec + 255) / 256, 1184);
    push_chunks_kernel<<<blocks, 256, 0, at::cuda::getCurrentCUDAStream()>>>(reinterpret_cast<const uint4*>(src.data_ptr()), dst, chunk_bytes / 16,
                                                                           dst_stride_bytes / 16, total_vec);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// out: contiguous [chunks, chunk_elems] (bf16 or fp32).  out[c] = sum over j of the bf16 piece at
// src_ptrs[j] + (src_offset_elems + c * src_stride_elems) elements.
void tp_reduce_chunks(std::vector<int64_t> src_ptrs, at::Tensor out, int64_t chunks, int64_t src_stride_elems, int64_t src_offset_elems) {
    TORCH_CHECK(out.is_cuda() && out.is_contiguous() && (out.scalar_type() == at::kFloat || out.scalar_type() == at::kBFloat16),
                "tp_reduce_chunks: contiguous fp32 or bf16 output required");
    TORCH_CHECK(chunks >= 1 && out.numel() % chunks == 0, "tp_reduce_chunks: the output does not split into equal chunks");
    const int64_t chunk_elems = out.numel() / chunks;
    TORCH_CHECK(chunk_elems % 8 == 0 && src_stride_elems % 8 == 0 && src_offset_elems % 8 == 0, "tp_reduce_chunks: 8-element granularity required");
    TORCH_CHECK(!src_ptrs.empty() && (int)src_ptrs.size() <= comm::kMaxWorld, "tp_reduce_chunks: 1..16 sources");
    const c10::cuda::CUDAGuard guard(out.device());
    ChunkPeers src{};
    src.n = (int)src_ptrs.size();
    for (int j = 0; j < src.n; ++j) {
        TORCH_CHECK(src_ptrs[j] % 16 == 0, "tp_reduce_chunks: sources must be 16-byte aligned");
        src.p[j] = reinterpret_cast<uint8_t*>(src_ptrs[j] + src_offset_elems * 2);
    }
    const long long total_vec = out.numel() / 8;
    const unsigned blocks = (unsigned)std::min<long long>((total_vec + 255) / 256, 1184);
    cudaStream_t st = at::cuda::getCurrentCUDAStream();
    if (out.scalar_type() == at::kFloat)
        reduce_chunks_kernel<float><<<blocks, 256, 0, st>>>(src, out.data_ptr<float>(), chunk_elems / 8, src_stride_elems / 8, total_vec);
    else
        reduce_chunks_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(src, reinterpret_cast<__nv_bfloat16*>(out.data_ptr()), chunk_elems / 8,
                                                                   src_stride_elems / 8, total_vec);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
}

void tp_barrier(std::vector<int64_t> sig_ptrs, int64_t rank, int64_t epoch, at::Tensor status, double timeout_s) {
    const int world = (int)sig_ptrs.size();
    TORCH_CHECK(world >= 1 && world <= comm::kMaxWorld, "tp_barrier: bad world size");
    TORCH_CHECK(status.is_cuda() && status.scalar_type() == at::kInt && status.numel() >= 4, "tp_barrier: status must be int32[4]");
    const c10::cuda::CUDAGuard guard(status.device());
    comm::PeerPtrs pp{};
    for (int j = 0; j < world; ++j) pp.sig[j] = reinterpret_cast<uint32_t*>(sig_ptrs[j]);
    const long long timeout_ns = (long long)(timeout_s * 1e9) + 1000;
    tp_barrier_kernel<<<1, 32, 0, at::cuda::getCurrentCUDAStream()>>>(pp, (int)rank, world, (uint32_t)epoch,
                                                                     reinterpret_cast<comm::CommStatus*>(status.data_ptr<int>()), timeout_ns);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
}

}  // namespace sjb200

TORCH_LIBRARY_FRAGMENT(sjb200, m) {
    m.def("spike_gemm(int[] a_ptrs, int a_pitch, int M, int K, Tensor w, int rows_per_t, int rows_per_src, int rank, int[] push_ptrs, int slot_elems) -> Tensor");
    m.def("lif_pack(Tensor x, int out_ptr, int pitch, float tau, float v_th) -> ()");
    m.def("rmsnorm_lif_pack(Tensor h, Tensor weight, int[] out_ptrs, int pitch, float eps, float tau, float v_th) -> ()");
    m.def("tp_reduce_residual(Tensor(a!) h, int stage_ptr, int slot_elems, int world) -> ()");
    m.def("tp_barrier(int[] sig_ptrs, int rank, int epoch, Tensor(a!) status, float timeout_s) -> ()");
    m.def("tp_push_chunks(Tensor src, int[] dst_ptrs, int chunks, int dst_stride_bytes, int dst_offset_bytes) -> ()");
    m.def("tp_reduce_chunks(int[] src_ptrs, Tensor(a!) out, int chunks, int src_stride_elems, int src_offset_elems) -> ()");
}
TORCH_LIBRARY_IMPL(sjb200, CUDA, m) {
    m.impl("spike_gemm", &sjb200::spike_gemm);
    m.impl("lif_pack", &sjb200::lif_pack);
    m.impl("rmsnorm_lif_pack", &sjb200::rmsnorm_lif_pack);
    m.impl("tp_reduce_residual", &sjb200::tp_reduce_residual);
    m.impl("tp_barrier", &sjb200::tp_barrier);
    m.impl("tp_push_chunks", &sjb200::tp_push_chunks);
    m.impl("tp_reduce_chunks", &sjb200::tp_reduce_chunks);
}
