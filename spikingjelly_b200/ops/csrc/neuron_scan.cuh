// Multi-step spiking-neuron scan (charge -> fire -> reset over T) and its BPTT
// backward, as one kernel each.  One thread owns V consecutive neurons and keeps
// their membrane potential in registers for the whole sequence.
//
// Forward writes spikes (and optionally v_seq / bit-packed spikes).  It saves no
// intermediate for backward: backward re-runs the recurrence from x_seq in
// register-resident chunks of TC steps (membrane potential at chunk boundaries is
// checkpointed in fp32 when T > TC) and then walks the chunk in reverse.
//
// Arithmetic is fp32 in the exact operation order of the eager formulas
//   IF : h = v + x
//   LIF: h = v + (x - (v - vr)) / tau            (decay_input)
//        h = v - (v - vr) / tau + x              (no decay_input)
//   PLIF: same with "* r", r = sigmoid(w) read from device memory
//   QIF: h = v + (x + a0 (v - v_rest)(v - v_c)) / tau
//   EIF: h = v + (x + v_rest - v + dT exp((v - theta_rh)/dT)) / tau
//   s = [h - v_th >= 0];  v = soft ? h - s v_th : s v_reset + (1 - s) h
// written with the non-contracting __f*_rn intrinsics, so fp32 spikes are
// bit-identical to PyTorch eager ops (EIF up to the accuracy of expf).
// Behavioural parity: spikingjelly/activation_based/functional/neuron.py:173-228,
// 242-312, 797-933, 1215-1297, 315-488; BPTT as in
// triton_kernel/neuron_kernel/lif.py:369-391 and plif.py:323-357.
#pragma once
#include "common.cuh"
#include "surrogate.cuh"

namespace sjb200 {

enum NeuronKind : int { NK_IF = 0, NK_LIF_DI = 1, NK_LIF_NDI = 2, NK_PLIF_DI = 3, NK_PLIF_NDI = 4, NK_QIF = 5, NK_EIF = 6 };

struct ScanParams {
    // sizes
    int T;
    long long N;
    // neuron
    int kind;
    float tau;          // LIF/QIF/EIF time constant
    float q0, q1, q2;   // QIF: a0, v_rest, v_c   EIF: delta_T, theta_rh, v_rest
    const float* r_ptr; // PLIF: device scalar r = sigmoid(w)
    float v_th, v_reset;
    int soft_reset;
    // surrogate / BPTT
    int sg_id;
    float sg_p0, sg_p1;
    int detach_reset;
    // initial state: tensor (may be null) or scalar
    const void* v_init;
    float v_init_scalar;
};

struct Neuron {
    int kind;
    float tau, r, q0, q1, q2, vr, v_th, v_reset;
    int soft;

    __device__ __forceinline__ Neuron(const ScanParams& p)
        : kind(p.kind), tau(p.tau), q0(p.q0), q1(p.q1), q2(p.q2), v_th(p.v_th), v_reset(p.v_reset), soft(p.soft_reset) {
        vr = p.soft_reset ? 0.0f : p.v_reset;
        r = (p.kind == NK_PLIF_DI || p.kind == NK_PLIF_NDI) ? *p.r_ptr : 0.0f;
    }
    // The round-to-nearest intrinsics are never contracted into FMAs, so every
    // intermediate is rounded exactly like a separate eager fp32 op.
    __device__ __forceinline__ float charge(float x, float v) const {
        switch (kind) {
        case NK_IF: return __fadd_rn(v, x);
        case NK_LIF_DI: return __fadd_rn(v, __fdiv_rn(__fsub_rn(x, __fsub_rn(v, vr)), tau));
        case NK_LIF_NDI: return __fadd_rn(__fsub_rn(v, __fdiv_rn(__fsub_rn(v, vr), tau)), x);
        case NK_PLIF_DI: return __fadd_rn(v, __fmul_rn(__fsub_rn(x, __fsub_rn(v, vr)), r));
        case NK_PLIF_NDI: return __fadd_rn(__fsub_rn(v, __fmul_rn(__fsub_rn(v, vr), r)), x);
        case NK_QIF:
            return __fadd_rn(v, __fdiv_rn(__fadd_rn(x, __fmul_rn(__fmul_rn(q0, __fsub_rn(v, q1)), __fsub_rn(v, q2))), tau));
        case NK_EIF:
            return __fadd_rn(v, __fdiv_rn(__fadd_rn(__fsub_rn(__fadd_rn(x, q2), v),
                                                   __fmul_rn(q0, expf(__fdiv_rn(__fsub_rn(v, q1), q0)))), tau));
        default: return __fadd_rn(v, x);
        }
    }
    __device__ __forceinline__ float fire(float h) const { return (__fsub_rn(h, v_th) >= 0.0f) ? 1.0f : 0.0f; }
    __device__ __forceinline__ float reset(float h, float s) const {
        return soft ? __fsub_rn(h, __fmul_rn(s, v_th)) : __fadd_rn(__fmul_rn(s, v_reset), __fmul_rn(__fsub_rn(1.0f, s), h));
    }
    // dh/dv at membrane potential v (before charging)
    __device__ __forceinline__ float dh_dv(float v) const {
        switch (kind) {
        case NK_IF: return 1.0f;
        case NK_LIF_DI: case NK_LIF_NDI: return 1.0f - 1.0f / tau;
        case NK_PLIF_DI: case NK_PLIF_NDI: return 1.0f - r;
        case NK_QIF: return 1.0f + q0 * (2.0f * v - q1 - q2) / tau;
        case NK_EIF: return 1.0f + (expf((v - q1) / q0) - 1.0f) / tau;
        default: return 1.0f;
        }
    }
    __device__ __forceinline__ float dh_dx() const {
        switch (kind) {
        case NK_LIF_DI: case NK_QIF: case NK_EIF: return 1.0f / tau;
        case NK_PLIF_DI: return r;
        default: return 1.0f;
        }
    }
};

// ------------------------------------------------------------------- forward
// spike_seq [T,N] (TO), v_last [N] (TIN), optional v_seq [T,N] (TIN),
// optional packed [T, ceil(N/32)] (bit i of word j = neuron 32 j + i),
// optional ckpt [ceil(T/TC)-1, N] fp32 (membrane potential after step (j+1)*TC-1).
template <typename TIN, typename TO, int V, int TC>
__global__ void __launch_bounds__(256)
scan_forward_kernel(ScanParams p, const TIN* __restrict__ x_seq, TO* __restrict__ spike_seq,
                    TIN* __restrict__ v_last, TIN* __restrict__ v_seq, uint32_t* __restrict__ packed,
                    float* __restrict__ ckpt) {
    const long long gtid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long n0 = gtid * V;
    const bool active = n0 < p.N;
    const Neuron nrn(p);
    const long long words = (p.N + 31) / 32;

    float v[V];
    if (active && p.v_init != nullptr) {
        load_vec<TIN, V>(reinterpret_cast<const TIN*>(p.v_init) + n0, v);
    } else {
#pragma unroll
        for (int j = 0; j < V; ++j) v[j] = p.v_init_scalar;
    }

    for (int t0 = 0; t0 < p.T; t0 += TC) {
        float x[TC][V];
#pragma unroll
        for (int i = 0; i < TC; ++i) {
            if (active && t0 + i < p.T) load_vec_stream<TIN, V>(x_seq + (long long)(t0 + i) * p.N + n0, x[i]);
        }
#pragma unroll
        for (int i = 0; i < TC; ++i) {
            if (t0 + i < p.T) {
                float s[V];
                uint32_t bits = 0;
#pragma unroll
                for (int j = 0; j < V; ++j) {
                    const float h = nrn.charge(x[i][j], v[j]);
                    s[j] = nrn.fire(h);
                    v[j] = nrn.reset(h, s[j]);
                    bits |= (s[j] != 0.0f ? 1u : 0u) << j;
                }
                const long long off = (long long)(t0 + i) * p.N + n0;
                if (active) {
                    store_vec<TO, V>(spike_seq + off, s);
                    if (v_seq != nullptr) store_vec<TIN, V>(v_seq + off, v);
                }
                if (packed != nullptr) {  // uniform branch: every lane of the warp takes part
                    if (!active) bits = 0;
                    constexpr int LPW = 32 / V;  // lanes per 32-bit word
                    uint32_t word = bits << ((threadIdx.x % LPW) * V);
#pragma unroll
                    for (int o = 1; o < LPW; o <<= 1) word |= __shfl_xor_sync(0xffffffffu, word, o);
                    if (active && (threadIdx.x % LPW) == 0) packed[(long long)(t0 + i) * words + n0 / 32] = word;
                }
            }
        }
        if (ckpt != nullptr && active && t0 + TC < p.T) {
            store_vec<float, V>(ckpt + (long long)(t0 / TC) * p.N + n0, v);
        }
    }
    if (active && v_last != nullptr) store_vec<TIN, V>(v_last + n0, v);
}

// ------------------------------------------------------------------ backward
// grad_x_seq [T,N] (TIN); optional grad_v_init [N] (TIN); PLIF: block partial sums of
// dL/dr go to partial[gridDim.x], the last block to finish (ticket counter) adds them
// in index order into grad_r[0] — a deterministic single-launch reduction.
template <typename TIN, typename TG, int V, int TC>
__global__ void __launch_bounds__(256)
scan_backward_kernel(ScanParams p, const TIN* __restrict__ x_seq, const TG* __restrict__ grad_spike_seq,
                     const TIN* __restrict__ grad_v_last, const TIN* __restrict__ grad_v_seq,
                     const float* __restrict__ ckpt, TIN* __restrict__ grad_x_seq, TIN* __restrict__ grad_v_init,
                     float* __restrict__ grad_r, float* __restrict__ partial, unsigned int* __restrict__ ticket) {
    const long long gtid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long n0 = gtid * V;
    const bool active = n0 < p.N;
    const Neuron nrn(p);
    const bool plif = (p.kind == NK_PLIF_DI || p.kind == NK_PLIF_NDI);
    const bool need_v = plif || p.kind == NK_QIF || p.kind == NK_EIF;
    const float dhdx = nrn.dh_dx();

    float c[V];     // dL/dv_t flowing in from step t+1
    float gr = 0.0f;
    if (active && grad_v_last != nullptr) {
        load_vec<TIN, V>(grad_v_last + n0, c);
    } else {
#pragma unroll
        for (int j = 0; j < V; ++j) c[j] = 0.0f;
    }

    const int n_chunks = (p.T + TC - 1) / TC;
    for (int ck = n_chunks - 1; ck >= 0; --ck) {
        const int t0 = ck * TC;
        float v0[V];  // membrane potential entering the chunk
        if (!active) {
#pragma unroll
            for (int j = 0; j < V; ++j) v0[j] = 0.0f;
        } else if (ck > 0) {
            load_vec<float, V>(ckpt + (long long)(ck - 1) * p.N + n0, v0);
        } else if (p.v_init != nullptr) {
            load_vec<TIN, V>(reinterpret_cast<const TIN*>(p.v_init) + n0, v0);
        } else {
#pragma unroll
            for (int j = 0; j < V; ++j) v0[j] = p.v_init_scalar;
        }
        // recompute h for the chunk (h overwrites x in place)
        float h[TC][V];
#pragma unroll
        for (int i = 0; i < TC; ++i) {
            if (active && t0 + i < p.T) load_vec_stream<TIN, V>(x_seq + (long long)(t0 + i) * p.N + n0, h[i]);
        }
        {
            float v[V];
#pragma unroll
            for (int j = 0; j < V; ++j) v[j] = v0[j];
#pragma unroll
            for (int i = 0; i < TC; ++i) {
                if (t0 + i < p.T) {
#pragma unroll
                    for (int j = 0; j < V; ++j) {
                        const float hh = nrn.charge(h[i][j], v[j]);
                        h[i][j] = hh;
                        v[j] = nrn.reset(hh, nrn.fire(hh));
                    }
                }
            }
        }
        // reverse walk
#pragma unroll
        for (int i = TC - 1; i >= 0; --i) {
            if (t0 + i < p.T) {
                const long long off = (long long)(t0 + i) * p.N + n0;
                float gs[V], gv[V], gx[V];
                if (active) {
                    load_vec_stream<TG, V>(grad_spike_seq + off, gs);
                    if (grad_v_seq != nullptr) load_vec_stream<TIN, V>(grad_v_seq + off, gv);
                }
#pragma unroll
                for (int j = 0; j < V; ++j) {
                    if (!active) { gs[j] = 0.0f; }
                    const float hh = h[i][j];
                    const float s = nrn.fire(hh);
                    const float sg = surrogate_grad(p.sg_id, hh - p.v_th, p.sg_p0, p.sg_p1);
                    const float g = c[j] + ((active && grad_v_seq != nullptr) ? gv[j] : 0.0f);
                    float dv_dh;  // d v_t / d h_t through the reset
                    if (p.soft_reset) dv_dh = 1.0f - (p.detach_reset ? 0.0f : p.v_th * sg);
                    else dv_dh = (1.0f - s) + (p.detach_reset ? 0.0f : (p.v_reset - hh) * sg);
                    const float gh = gs[j] * sg + g * dv_dh;
                    float vprev = 0.0f;
                    if (need_v) {
                        if (i == 0) vprev = v0[j];
                        else { const float hp = h[i > 0 ? i - 1 : 0][j]; vprev = nrn.reset(hp, nrn.fire(hp)); }
                    }
                    if (plif) gr += (p.kind == NK_PLIF_DI) ? gh * (hh - vprev) / nrn.r : gh * (nrn.vr - vprev);
                    c[j] = gh * nrn.dh_dv(vprev);
                    gx[j] = gh * dhdx;
                }
                if (active) store_vec<TIN, V>(grad_x_seq + off, gx);
            }
        }
    }
    if (active && grad_v_init != nullptr) store_vec<TIN, V>(grad_v_init + n0, c);

    if (plif) {  // uniform
        __shared__ float warp_part[8];
        __shared__ bool last_block;
        gr = warp_sum(active ? gr : 0.0f);
        if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = gr;
        __syncthreads();
        if (threadIdx.x == 0) {
            float tot = 0.0f;
            for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += warp_part[w];
            partial[blockIdx.x] = tot;
            __threadfence();
            const unsigned int done = atomicAdd(ticket, 1u);
            last_block = (done == gridDim.x - 1);
        }
        __syncthreads();
        if (last_block) {
            __threadfence();
            // fixed-order tree over the block partials: thread k sums k, k+256, ...
            float acc = 0.0f;
            for (unsigned int b = threadIdx.x; b < gridDim.x; b += blockDim.x) acc += __ldcg(partial + b);
            acc = warp_sum(acc);
            __syncthreads();
            if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = acc;
            __syncthreads();
            if (threadIdx.x == 0) {
                float tot = 0.0f;
                for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += warp_part[w];
                grad_r[0] = tot;
                *ticket = 0u;  // ready for the next launch
            }
        }
    }
}

}  // namespace sjb200
