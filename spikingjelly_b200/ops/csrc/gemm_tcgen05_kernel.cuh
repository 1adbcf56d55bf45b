// Kernel side of the tcgen05 GEMM family (included by gemm_tcgen05.cu and conv_tcgen05.cu).
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
#pragma once
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
constexpr int kThreads = 320;
constexpr int kSpinPolls = 512;            // non-suspending probes of a ring barrier before falling back to the bounded, suspending wait
constexpr int kWarpStageBytes = 32 * 64;   // one epilogue warp's staging buffer: 32 rows x 32 16-bit columns   // 10 warps: producer, mma, 2 x 4 epilogue (each group of four drains half of the columns)

template <int BN, int STAGES>
struct SmemLayout {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
    static constexpr int OUT_OFFSET = BAR_OFFSET + 1024;    // epilogue staging: 8 warps x 2 x [32 rows][32 cols] 16-bit
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
    const float* alpha;     // optional device scalar multiplied into the result (an fp8 de-quantisation scale, or the product of two)
    const float* alpha2;    // optional second device scalar (used only together with `alpha`)
    const float* bias;      // optional fp32 vector [N] added to every row (by split 0 when the contraction is split)
    float* stats;           // optional [ceil(M / 128) * 4][2][N]: per-column sum and sum of squares of the rounded
                            // 16-bit result over each 32-row slice (batch-norm statistics without re-reading D)
};

// Geometry of an implicit-GEMM convolution operand (LOADER != 0): one operand is gathered from an NHWC tensor by TMA
// im2col loads instead of being read as a matrix.
//   LOADER 1 (forward, data gradient): A[m, (tap, c)] = src[pixel(m) + tap offset][c]; m walks the traversal grid
//            (img, i < Ht, j < Wt) with position (base_h + i * step_h, base_w + j * step_w); the contraction runs over
//            taps_h x taps_w taps (offset tap * dil) and the source's CA channels in blocks of 64.  B is the filter
//            [Cout][R * S * Cin]: K-major rows for the forward pass, MN-major (rows = Cout) for the data gradient;
//            its tap is (wr0 + wr_step * th) * S + (ws0 + ws_step * tw).
//   LOADER 2 (weight gradient): B[pixel, (tap, c)] gathered the same way (64 pixels per k-block), A = dY [pixels][Cout]
//            MN-major; the contraction runs over the pixels.
// scatter != 0: output row m = (img, i, j) is stored at pixel (img, i * out_mul_h + out_add_h, j * out_mul_w + out_add_w)
// of an [*, out_H, out_W, ldd] tensor instead of at row m (data gradient of a strided convolution, one launch per
// parity class of input pixels).
struct ConvGeom {
    int Ht, Wt;
    int base_h, base_w, step_h, step_w;
    int taps_h, taps_w, dil_h, dil_w;
    int CA;                 // channels of the gathered tensor (multiple of 64)
    int CN;                 // LOADER 1 with MN-major B: filter columns per tap (= Cin); LOADER 2: channels per tap
    int wr0, wr_step, ws0, ws_step, S;
    int scatter, out_H, out_W, out_mul_h, out_mul_w, out_add_h, out_add_w;
};

// Epilogue of one output tile for one warp: drains NCHUNK chunks of 32 accumulator columns (this warp's 32 TMEM lanes =
// 32 output rows) starting at chunk `c_begin`.  The TMEM load of chunk i + 1 is in flight while chunk i is converted
// and stored.  16-bit results are staged in a buffer that belongs to this warp alone (32 rows x 64 bytes, 16-byte
// chunks XOR-swizzled by (row >> 1) & 3 = the TMA 64-byte swizzle) and written by a TMA store of a 32 x 32 box:
// full sectors, clipped at the matrix edges, asynchronous, and no barrier between warps.  `oc` counts this warp's
// staged chunks (two buffers alternate; a buffer is reused once the store that read it has finished reading).
template <int NCHUNK, int LOADER>
__device__ __forceinline__ void drain_accumulator(uint32_t taddr, int c_begin, int m0, int n0, int split, int quarter, int lane,
                                                  void* __restrict__ Dptr, const GemmArgs& g, const ConvGeom& cg, float alpha,
                                                  const CUtensorMap* tmD, uint8_t* warp_stage, uint32_t& oc) {
    const int row0 = m0 + quarter * 32, row = row0 + lane;
    uint32_t r[32];
    tmem_ld_32x32(taddr + c_begin * 32, r);
#pragma unroll
    for (int ci = 0; ci < NCHUNK; ++ci) {
        const int c = c_begin + ci;
        tmem_ld_wait();
        uint32_t cur[32];
#pragma unroll
        for (int q = 0; q < 32; ++q) cur[q] = r[q];
        if (ci + 1 < NCHUNK) tmem_ld_32x32(taddr + (c + 1) * 32, r);      // next chunk travels while this one is stored
        if (g.alpha != nullptr) {
#pragma unroll
            for (int q = 0; q < 32; ++q) cur[q] = __float_as_uint(__uint_as_float(cur[q]) * alpha);
        }
        const int col0 = n0 + c * 32;
        if (g.bias != nullptr && split == 0) {
#pragma unroll
            for (int q = 0; q < 32; ++q)
                if (col0 + q < g.N) cur[q] = __float_as_uint(__uint_as_float(cur[q]) + __ldg(g.bias + col0 + q));
        }
        if (g.out_f32) {
            // split-K partial sums / fp32 results: straight from registers, one 128-byte run per row
            if (row < g.M && col0 < g.N) {
                float* dst = reinterpret_cast<float*>(Dptr) + ((size_t)split * g.M + row) * g.ldd + col0;
                if (col0 + 32 <= g.N) {
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        reinterpret_cast<uint4*>(dst)[q] = make_uint4(cur[4 * q], cur[4 * q + 1], cur[4 * q + 2], cur[4 * q + 3]);
                } else {
#pragma unroll
                    for (int q = 0; q < 32; ++q)
                        if (col0 + q < g.N) dst[q] = __uint_as_float(cur[q]);
                }
            }
            continue;
        }
        uint32_t w[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
            const float lo = __uint_as_float(cur[2 * e]), hi = __uint_as_float(cur[2 * e + 1]);
            if (g.out_bf16) { __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi); w[e] = *reinterpret_cast<uint32_t*>(&v); }
            else { __half2 v = __floats2half2_rn(lo, hi); w[e] = *reinterpret_cast<uint32_t*>(&v); }
        }
        if constexpr (LOADER == 1) {
            if (cg.scatter) {
                // strided data gradient: this row is one input pixel of the launch's parity class
                if (row < g.M && col0 + 32 <= g.N) {
                    const int per_img = cg.Ht * cg.Wt;
                    const int img = row / per_img, rem = row - img * per_img, i = rem / cg.Wt, j = rem - i * cg.Wt;
                    const size_t pix = ((size_t)img * cg.out_H + (i * cg.out_mul_h + cg.out_add_h)) * cg.out_W +
                                       (j * cg.out_mul_w + cg.out_add_w);
                    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(Dptr) + pix * g.ldd + col0);
#pragma unroll
                    for (int q = 0; q < 4; ++q) dst[q] = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
                }
                continue;
            }
        }
        if (col0 >= g.N) continue;                              // nothing of this box lies inside the matrix (warp-uniform)
        uint8_t* stage_buf = warp_stage + (oc & 1) * kWarpStageBytes;
        if (oc >= 2) {
            if (lane == 0) tma_store_wait_read<1>();               // the store that last read this buffer is done
            __syncwarp();
        }
        ++oc;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int chunk = q ^ ((lane >> 1) & 3);
            *reinterpret_cast<uint4*>(stage_buf + lane * 64 + chunk * 16) = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
            // rows past M are clipped by the TMA unit; a box that starts past M is not issued at all (its rows are zero and
            // still feed the column sums below, so that every statistics slot is written)
            if (row0 < g.M) tma_store_2d(tmD, stage_buf, col0, row0);
            tma_store_commit();
        }
        if (g.stats != nullptr) {
            // Column sums over this warp's 32 staged rows (the rounded values a batch norm will read).
            // Lane = (column pair, row half); the upper half walks its rows one step ahead so that the
            // two halves hit different 64-byte halves of a bank line.
            const int cp = lane & 15, hi = lane >> 4;
            float s1a = 0.f, s1b = 0.f, s2a = 0.f, s2b = 0.f;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int rr = hi * 16 + ((i + hi) & 15);
                const int chunk = (cp >> 2) ^ ((rr >> 1) & 3);
                const uint32_t v = *reinterpret_cast<const uint32_t*>(stage_buf + rr * 64 + chunk * 16 + (cp & 3) * 4);
                float lo, up;
                if (g.out_bf16) { lo = __uint_as_float(v << 16); up = __uint_as_float(v & 0xffff0000u); }
                else { const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&v)); lo = f.x; up = f.y; }
                s1a += lo; s1b += up; s2a = fmaf(lo, lo, s2a); s2b = fmaf(up, up, s2b);
            }
            s1a += __shfl_xor_sync(0xffffffffu, s1a, 16); s1b += __shfl_xor_sync(0xffffffffu, s1b, 16);
            s2a += __shfl_xor_sync(0xffffffffu, s2a, 16); s2b += __shfl_xor_sync(0xffffffffu, s2b, 16);
            const int col = col0 + cp * 2;
            if (hi == 0 && col < g.N) {
                float* dst = g.stats + ((size_t)((m0 / BM) * 4 + quarter) * 2) * g.N + col;
                *reinterpret_cast<float2*>(dst) = make_float2(s1a, s1b);
                *reinterpret_cast<float2*>(dst + g.N) = make_float2(s2a, s2b);
            }
        }
    }
}

// ES: operand element size in bytes (2: fp16 / bf16, 1: fp8).  A k-block is always one 128-byte
// swizzle row, i.e. 128 / ES elements, and is consumed by four MMAs of 32 bytes of K each.
template <int BN, int STAGES, bool A_MN, bool B_MN, int ES = 2, int LOADER = 0>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ CUtensorMap tmD, void* __restrict__ Dptr, GemmArgs g, KernelStatus* __restrict__ status,
            const ConvGeom cg) {
    static_assert(LOADER == 0 || ES == 2, "implicit-GEMM operands are 16-bit");
    static_assert(LOADER != 1 || !A_MN, "the gathered A operand is K-major");
    static_assert(LOADER != 2 || (A_MN && B_MN), "weight gradient: both operands are MN-major");
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
    const float alpha = g.alpha != nullptr ? __ldg(g.alpha) * (g.alpha2 != nullptr ? __ldg(g.alpha2) : 1.0f) : 1.0f;

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

    // The producer and the MMA issuer are single threads: their loops run at one dependent instruction every few
    // cycles, so the instruction count per k-block IS the time per k-block when tiles are small.  Both keep the ring
    // position (stage, phase, shared-memory addresses, descriptor words) in registers and update it by increments;
    // nothing in the k-block loops divides or rebuilds a 64-bit descriptor.
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t full_base = smem_u32(full_bar), empty_base = smem_u32(empty_bar);
    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;                         // ring position, carried across tiles
            for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x) {
                const int split = tile / tiles_mn, mn = tile % tiles_mn;
                int tm, tn;
                tile_coords(mn, tiles_m, tiles_n, tm, tn);
                const int m0 = tm * BM, n0 = tn * BN;
                const int kb0 = split * g.kb_per_split;
                const int kb1 = min(kb_total, kb0 + g.kb_per_split);
                // implicit-GEMM operands: where this tile's first row sits on the traversal grid (LOADER 1), or which
                // (tap, channel) each 64-column chunk of the tile is (LOADER 2)
                int cv_img = 0, cv_h = 0, cv_w = 0, cv_valid = BN / 64;
                int cv_chan[BN / 64], cv_offw[BN / 64], cv_offh[BN / 64];
                int tap_h = 0, tap_w = 0, chan = 0;                // LOADER 1: position inside the contraction
                int px_img = 0, px_i = 0, px_j = 0;                // LOADER 2: first pixel of the k-block on the traversal grid
                if constexpr (LOADER == 1) {
                    const int per_img = cg.Ht * cg.Wt;
                    cv_img = m0 / per_img;
                    const int rem = m0 - cv_img * per_img, i = rem / cg.Wt;
                    cv_h = cg.base_h + i * cg.step_h;
                    cv_w = cg.base_w + (rem - i * cg.Wt) * cg.step_w;
                    const int cpb = cg.CA / 64, tap = kb0 / cpb;
                    chan = (kb0 - tap * cpb) * 64;
                    tap_h = tap / cg.taps_w;
                    tap_w = tap - tap_h * cg.taps_w;
                }
                if constexpr (LOADER == 2) {
                    cv_valid = 0;
#pragma unroll
                    for (int c = 0; c < BN / 64; ++c) {
                        const int nn = n0 + c * 64;
                        const int tap = nn / cg.CN, th = tap / cg.taps_w;
                        cv_chan[c] = nn - tap * cg.CN;
                        cv_offh[c] = th * cg.dil_h;
                        cv_offw[c] = (tap - th * cg.taps_w) * cg.dil_w;
                        if (nn < g.N) cv_valid = c + 1;
                    }
                    const int p0 = kb0 * BK, per_img = cg.Ht * cg.Wt;
                    px_img = p0 / per_img;
                    const int rem = p0 - px_img * per_img;
                    px_i = rem / cg.Wt;
                    px_j = rem - px_i * cg.Wt;
                }
                int k0 = kb0 * BKE;
                for (int kb = kb0; kb < kb1; ++kb) {
                    uint64_t* const fb = full_bar + stage;
                    if (!mbar_spin(empty_bar + stage, phase ^ 1, kSpinPolls) && !mbar_wait_bounded(empty_bar + stage, phase ^ 1)) {
                        report(status, WAIT_EMPTY, stage); *abort_flag = 1; break;
                    }
                    uint8_t* sa = smem + stage * L::STAGE_BYTES;
                    uint8_t* sb = sa + L::A_BYTES;
                    if constexpr (LOADER == 1) {
                        mbar_expect_tx(fb, L::STAGE_BYTES);
                        tma_load_im2col_4d(sa, &tmA, chan, cv_w, cv_h, cv_img, (uint16_t)(tap_w * cg.dil_w), (uint16_t)(tap_h * cg.dil_h), fb);
                        const int wtap = (cg.wr0 + cg.wr_step * tap_h) * cg.S + (cg.ws0 + cg.ws_step * tap_w);
                        if (B_MN) {
#pragma unroll
                            for (int c = 0; c < BN / 64; ++c)
                                tma_load_2d(sb + c * (BK * 128), &tmB, wtap * cg.CN + n0 + c * 64, chan, fb);
                        } else {
                            tma_load_2d(sb, &tmB, wtap * cg.CA + chan, n0, fb);
                        }
                        chan += 64;
                        if (chan == cg.CA) { chan = 0; if (++tap_w == cg.taps_w) { tap_w = 0; ++tap_h; } }
                    } else if constexpr (LOADER == 2) {
                        mbar_expect_tx(fb, L::A_BYTES + cv_valid * (BK * 128));
                        const int ph0 = cg.base_h + px_i * cg.step_h, pw0 = cg.base_w + px_j * cg.step_w;
#pragma unroll
                        for (int c = 0; c < BM / 64; ++c) tma_load_2d(sa + c * (BK * 128), &tmA, m0 + c * 64, kb * BK, fb);
#pragma unroll
                        for (int c = 0; c < BN / 64; ++c)
                            if (c < cv_valid)
                                tma_load_im2col_4d(sb + c * (BK * 128), &tmB, cv_chan[c], pw0, ph0, px_img, (uint16_t)cv_offw[c],
                                                   (uint16_t)cv_offh[c], fb);
                        px_j += BK;                                  // 64 pixels further along the traversal
                        while (px_j >= cg.Wt) { px_j -= cg.Wt; if (++px_i == cg.Ht) { px_i = 0; ++px_img; } }
                    } else {
                        mbar_expect_tx(fb, L::STAGE_BYTES);
                        if (A_MN) {
#pragma unroll
                            for (int c = 0; c < BM / 64; ++c) tma_load_2d(sa + c * (BK * 128), &tmA, m0 + c * 64, k0, fb);
                        } else {
                            tma_load_2d(sa, &tmA, k0, m0, fb);
                        }
                        if (B_MN) {
#pragma unroll
                            for (int c = 0; c < BN / 64; ++c) tma_load_2d(sb + c * (BK * 128), &tmB, n0 + c * 64, k0, fb);
                        } else {
                            tma_load_2d(sb, &tmB, k0, n0, fb);
                        }
                        k0 += BKE;
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            const uint32_t idesc = make_idesc_f16(g.ab_format, A_MN ? 1 : 0, B_MN ? 1 : 0, BM, BN);
            // Descriptor words.  High word: stride offset 1024 B, version 1, 128-byte swizzle.  Low word: start address >> 4
            // plus the leading-dimension offset (16 B for K-major; the distance between 64-element chunks for MN-major).
            constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
            constexpr uint32_t kLboA = A_MN ? ((BK * 128u) >> 4) : 1u, kLboB = B_MN ? ((BK * 128u) >> 4) : 1u;
            constexpr uint32_t kStepA = (A_MN ? UMMA_K * 128u : UMMA_K * 2u) >> 4, kStepB = (B_MN ? UMMA_K * 128u : UMMA_K * 2u) >> 4;
            const uint32_t a_lo0 = (smem_base >> 4) | (kLboA << 16), b_lo0 = ((smem_base + L::A_BYTES) >> 4) | (kLboB << 16);
            uint32_t stage = 0, phase = 0, a_lo = a_lo0, b_lo = b_lo0, tl = 0;
            for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x, ++tl) {
                const int split = tile / tiles_mn;
                const int kb0 = split * g.kb_per_split;
                const int kb1 = min(kb_total, kb0 + g.kb_per_split);
                const uint32_t acc = tl & 1, acc_ph = (tl >> 1) & 1;
                if (!mbar_wait_bounded(tempty_bar + acc, acc_ph ^ 1)) { report(status, WAIT_TMEM_EMPTY, tile); *abort_flag = 1; break; }
                fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * BN;
                uint32_t accumulate = 0;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_spin(full_bar + stage, phase, kSpinPolls) && !mbar_wait_bounded(full_bar + stage, phase)) {
                        report(status, WAIT_FULL, stage); *abort_flag = 1; break;
                    }
                    // no tcgen05 fence here: the operands were written by the TMA unit (async proxy) and published through
                    // the mbarrier this thread just observed; a fence per k-block would only serialise the MMA stream
#pragma unroll
                    for (int j = 0; j < BK / UMMA_K; ++j) {
                        // K-major: 16 elements = 32 B further along the swizzled row; MN-major: 16 k-rows of 128 B further down
                        if constexpr (ES == 2) mma_f16_ss_words(d_tmem, a_lo + j * kStepA, b_lo + j * kStepB, kDescHi, idesc, accumulate);
                        else mma_f8_ss_words(d_tmem, a_lo + j * kStepA, b_lo + j * kStepB, kDescHi, idesc, accumulate);
                        accumulate = 1;
                    }
                    mma_commit(empty_bar + stage);     // stage reusable once these MMAs have read it
                    a_lo += L::STAGE_BYTES >> 4;
                    b_lo += L::STAGE_BYTES >> 4;
                    if (++stage == STAGES) { stage = 0; phase ^= 1; a_lo = a_lo0; b_lo = b_lo0; }
                }
                mma_commit(tfull_bar + acc);       // accumulator complete
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        const int quarter = warp & 3;              // TMEM lane quarter this warp may read
        const int half = (warp - 2) >> 2;          // which half of the tile's columns this group of four warps drains
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
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
            drain_accumulator<BN / 64, LOADER>(taddr, half * (BN / 64), m0, n0, split, quarter, lane, Dptr, g, cg, alpha, &tmD,
                                               smem + L::OUT_OFFSET + (warp - 2) * 2 * kWarpStageBytes, oc);
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar + acc);
        }
        if (lane == 0) tma_store_wait_all<0>();                    // all output boxes written before the CTA retires
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
    const float alpha = g.alpha != nullptr ? __ldg(g.alpha) * (g.alpha2 != nullptr ? __ldg(g.alpha2) : 1.0f) : 1.0f;

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
            uint32_t stage = 0, phase = 0;
            const uint32_t full0 = map_to_cta(smem_u32(full_bar), 0);          // the full barriers live in the pair's first CTA
            for (int tile = pair; tile < total_tiles && !*abort_flag; tile += n_pairs) {
                const int split = tile / tiles_mn;
                int tm, tn;
                tile_coords(tile - split * tiles_mn, tiles_m, tiles_n, tm, tn);
                const int m0 = tm * (2 * BM) + (int)rank * BM;
                const int nb0 = tn * BN + (int)rank * (BN / 2);                    // this CTA's half of the B columns
                const int kb0 = split * g.kb_per_split, kb1 = min(kb_total, kb0 + g.kb_per_split);
                int k0 = kb0 * BKE;
                for (int kb = kb0; kb < kb1; ++kb, k0 += BKE) {
                    if (!mbar_spin(empty_bar + stage, phase ^ 1, kSpinPolls) && !mbar_wait_bounded(empty_bar + stage, phase ^ 1)) {
                        report(status, WAIT_EMPTY, stage); *abort_flag = 1; break;
                    }
                    uint8_t* sa = smem + stage * L::STAGE_BYTES;
                    uint8_t* sb = sa + L::A_BYTES;
                    if (first) mbar_expect_tx(full_bar + stage, 2 * L::STAGE_BYTES);
                    const uint32_t bar = full0 + stage * 8;
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
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer (first CTA only)
        if (lane == 0 && first) {
            const uint32_t idesc = make_idesc_f16(g.ab_format, A_MN ? 1 : 0, B_MN ? 1 : 0, 2 * BM, BN);
            constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
            constexpr uint32_t kLboA = A_MN ? ((BK * 128u) >> 4) : 1u, kLboB = B_MN ? ((BK * 128u) >> 4) : 1u;
            constexpr uint32_t kStepA = (A_MN ? UMMA_K * 128u : UMMA_K * 2u) >> 4, kStepB = (B_MN ? UMMA_K * 128u : UMMA_K * 2u) >> 4;
            const uint32_t smem_base = smem_u32(smem);
            const uint32_t a_lo0 = (smem_base >> 4) | (kLboA << 16), b_lo0 = ((smem_base + L::A_BYTES) >> 4) | (kLboB << 16);
            const uint32_t empty_self = smem_u32(empty_bar), empty_peer = map_to_cta(empty_self, 1);
            uint32_t stage = 0, phase = 0, a_lo = a_lo0, b_lo = b_lo0, tl = 0;
            for (int tile = pair; tile < total_tiles && !*abort_flag; tile += n_pairs, ++tl) {
                const int split = tile / tiles_mn;
                const int kb0 = split * g.kb_per_split, kb1 = min(kb_total, kb0 + g.kb_per_split);
                const uint32_t acc = tl & 1, acc_ph = (tl >> 1) & 1;
                if (!mbar_wait_bounded(tempty_bar + acc, acc_ph ^ 1)) { report(status, WAIT_TMEM_EMPTY, tile); *abort_flag = 1; break; }
                fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * BN;
                uint32_t accumulate = 0;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_spin(full_bar + stage, phase, kSpinPolls) && !mbar_wait_bounded(full_bar + stage, phase)) {
                        report(status, WAIT_FULL, stage); *abort_flag = 1; break;
                    }
                    // no tcgen05 fence here: the operands were written by the TMA unit (async proxy) and published through
                    // the mbarrier this thread just observed; a fence per k-block would only serialise the MMA stream
#pragma unroll
                    for (int j = 0; j < BK / UMMA_K; ++j) {
                        if constexpr (ES == 2) mma_f16_ss_pair_words(d_tmem, a_lo + j * kStepA, b_lo + j * kStepB, kDescHi, idesc, accumulate);
                        else mma_f8_ss_pair_words(d_tmem, a_lo + j * kStepA, b_lo + j * kStepB, kDescHi, idesc, accumulate);
                        accumulate = 1;
                    }
                    mma_commit_pair(empty_self + stage * 8);          // this CTA's stage is reusable ...
                    mma_commit_pair(empty_peer + stage * 8);          // ... and the partner's
                    a_lo += L::STAGE_BYTES >> 4;
                    b_lo += L::STAGE_BYTES >> 4;
                    if (++stage == STAGES) { stage = 0; phase ^= 1; a_lo = a_lo0; b_lo = b_lo0; }
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
        const uint32_t tempty_first = map_to_cta(smem_u32(tempty_bar), 0);
        uint32_t tl = 0, oc = 0;
        for (int tile = pair; tile < total_tiles && !*abort_flag; tile += n_pairs, ++tl) {
            const int split = tile / tiles_mn;
            int tm, tn;
            tile_coords(tile - split * tiles_mn, tiles_m, tiles_n, tm, tn);
            const int m0 = tm * (2 * BM) + (int)rank * BM, n0 = tn * BN;
            const uint32_t acc = tl & 1, acc_ph = (tl >> 1) & 1;
            bool ok = true;
            if (lane == 0) ok = mbar_wait_bounded(tfull_bar + acc, acc_ph);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) { if (lane == 0) { report(status, WAIT_TMEM_FULL, tile); *abort_flag = 1; } break; }
            fence_after_sync();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
            drain_accumulator<BN / 64, 0>(taddr, half * (BN / 64), m0, n0, split, quarter, lane, Dptr, g, ConvGeom{}, alpha, &tmD,
                                          smem + L::OUT_OFFSET + (warp - 2) * 2 * kWarpStageBytes, oc);
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tempty_first + acc * 8);      // the MMA thread lives in the first CTA
        }
        if (lane == 0) tma_store_wait_all<0>();
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
template <int BN, int STAGES, bool A_MN, bool B_MN, int ES = 2, int LOADER = 0>
void launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td, void* d, const GemmArgs& g,
            KernelStatus* st, int grid, cudaStream_t stream, const ConvGeom& cg = ConvGeom{}) {
    using L = SmemLayout<BN, STAGES>;
    auto kern = gemm_kernel<BN, STAGES, A_MN, B_MN, ES, LOADER>;
    static bool configured = false;
    if (!configured) {
        C10_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
        configured = true;
    }
    kern<<<grid, kThreads, L::TOTAL, stream>>>(ta, tb, td, d, g, st, cg);
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

}  // namespace sjb200
