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
    float inv_tau;      // fp32 reciprocal of the LIF/QIF/EIF time constant
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

// Dynamics of one neuron model, resolved at compile time.  Division by the python
// scalar tau is a multiplication by the fp32 reciprocal, exactly as PyTorch's CUDA
// `tensor / scalar` kernel evaluates it; the __f*_rn intrinsics are never contracted
// into FMAs, so every intermediate is rounded like a separate eager fp32 op.
template <int KIND>
struct Neuron {
    float inv_tau, r, inv_r, q0, q1, q2, vr, v_th, v_reset;
    int soft;

    __device__ __forceinline__ Neuron(const ScanParams& p)
        : inv_tau(p.inv_tau), q0(p.q0), q1(p.q1), q2(p.q2), v_th(p.v_th), v_reset(p.v_reset), soft(p.soft_reset) {
        vr = p.soft_reset ? 0.0f : p.v_reset;
        r = (KIND == NK_PLIF_DI || KIND == NK_PLIF_NDI) ? *p.r_ptr : 0.0f;
        inv_r = (KIND == NK_PLIF_DI) ? 1.0f / r : 0.0f;
    }
    __device__ __forceinline__ float charge(float x, float v) const {
        if constexpr (KIND == NK_IF) return __fadd_rn(v, x);
        else if constexpr (KIND == NK_LIF_DI) return __fadd_rn(v, __fmul_rn(__fsub_rn(x, __fsub_rn(v, vr)), inv_tau));
        else if constexpr (KIND == NK_LIF_NDI) return __fadd_rn(__fsub_rn(v, __fmul_rn(__fsub_rn(v, vr), inv_tau)), x);
        else if constexpr (KIND == NK_PLIF_DI) return __fadd_rn(v, __fmul_rn(__fsub_rn(x, __fsub_rn(v, vr)), r));
        else if constexpr (KIND == NK_PLIF_NDI) return __fadd_rn(__fsub_rn(v, __fmul_rn(__fsub_rn(v, vr), r)), x);
        else if constexpr (KIND == NK_QIF)
            return __fadd_rn(v, __fmul_rn(__fadd_rn(x, __fmul_rn(__fmul_rn(q0, __fsub_rn(v, q1)), __fsub_rn(v, q2))), inv_tau));
        else  // NK_EIF; q0 = delta_T, q1 = theta_rh, q2 = v_rest
            return __fadd_rn(v, __fmul_rn(__fadd_rn(__fsub_rn(__fadd_rn(x, q2), v),
                                                   __fmul_rn(q0, expf(__fmul_rn(__fsub_rn(v, q1), 1.0f / q0)))), inv_tau));
    }
    // h - v_th >= 0 and h >= v_th agree for all finite floats (x - y rounds to zero only if x == y)
    __device__ __forceinline__ bool fire(float h) const { return h >= v_th; }
    // soft: h - s v_th;  hard: s v_reset + (1 - s) h  (both reduce to these selects for finite h)
    __device__ __forceinline__ float reset(float h, bool s) const {
        return soft ? (s ? __fsub_rn(h, v_th) : h) : (s ? v_reset : h);
    }
    static constexpr bool kNeedsV = (KIND == NK_PLIF_DI || KIND == NK_PLIF_NDI || KIND == NK_QIF || KIND == NK_EIF);
    static constexpr bool kPlif = (KIND == NK_PLIF_DI || KIND == NK_PLIF_NDI);
    // dh/dv at membrane potential v (before charging)
    __device__ __forceinline__ float dh_dv(float v) const {
        if constexpr (KIND == NK_IF) return 1.0f;
        else if constexpr (KIND == NK_LIF_DI || KIND == NK_LIF_NDI) return 1.0f - inv_tau;
        else if constexpr (kPlif) return 1.0f - r;
        else if constexpr (KIND == NK_QIF) return 1.0f + q0 * (2.0f * v - q1 - q2) * inv_tau;
        else return 1.0f + (__expf((v - q1) / q0) - 1.0f) * inv_tau;
    }
    __device__ __forceinline__ float dh_dx() const {
        if constexpr (KIND == NK_LIF_DI || KIND == NK_QIF || KIND == NK_EIF) return inv_tau;
        else if constexpr (KIND == NK_PLIF_DI) return r;
        else return 1.0f;
    }
};

// ------------------------------------------------------------------- forward
// x_seq [T,N] (TIN: may be narrower than the rest, e.g. fp8-e4m3); spike_seq [T,N], v_last [N], optional v_seq [T,N] (TO),
// optional packed [T, ceil(N/32)] (bit i of word j = neuron 32 j + i),
// optional ckpt [ceil(T/TC)-1, N] fp32 (membrane potential after step (j+1)*TC-1).
// LEAN: the common training call, with everything optional compiled out: T is a multiple of TC (no
// per-step bounds predicates), scalar initial potential, no v_seq, no bit-packed output.
template <typename TIN, typename TO, int V, int TC, int KIND, bool LEAN = false>
__global__ void __launch_bounds__(256, 3)
scan_forward_kernel(ScanParams p, const TIN* __restrict__ x_seq, TO* __restrict__ spike_seq,
                    TO* __restrict__ v_last, TO* __restrict__ v_seq, uint32_t* __restrict__ packed,
                    float* __restrict__ ckpt) {
    const long long gtid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long n0 = gtid * V;
    if constexpr (LEAN) {
        if (n0 >= p.N) return;
        p.v_init = nullptr; v_seq = nullptr; packed = nullptr;
    }
    const bool active = LEAN ? true : (n0 < p.N);
    const Neuron<KIND> nrn(p);
    const long long words = (p.N + 31) / 32;

    float v[V];
    if (active && p.v_init != nullptr) {
        load_vec<TO, V>(reinterpret_cast<const TO*>(p.v_init) + n0, v);
    } else {
#pragma unroll
        for (int j = 0; j < V; ++j) v[j] = p.v_init_scalar;
    }

    for (int t0 = 0; t0 < p.T; t0 += TC) {
        Pack<TIN, V> xr[TC];   // all loads of the chunk are in flight before the first use
#pragma unroll
        for (int i = 0; i < TC; ++i) {
            if (active && (LEAN || t0 + i < p.T)) xr[i] = load_raw_stream<TIN, V>(x_seq + (long long)(t0 + i) * p.N + n0);
        }
#pragma unroll
        for (int i = 0; i < TC; ++i) {
            if (LEAN || t0 + i < p.T) {
                float x[V], s[V];
                unpack<TIN, V>(xr[i], x);
                uint32_t bits = 0;
#pragma unroll
                for (int j = 0; j < V; ++j) {
                    const float h = nrn.charge(x[j], v[j]);
                    const bool f = nrn.fire(h);
                    s[j] = f ? 1.0f : 0.0f;
                    v[j] = nrn.reset(h, f);
                    bits |= (f ? 1u : 0u) << j;
                }
                const long long off = (long long)(t0 + i) * p.N + n0;
                if (active) {
                    if (LEAN || spike_seq != nullptr) store_vec<TO, V>(spike_seq + off, s);      // null: bit-packed output only
                    if (v_seq != nullptr) store_vec<TO, V>(v_seq + off, v);
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
    if (active && v_last != nullptr) store_vec<TO, V>(v_last + n0, v);
}

// ------------------------------------------------------------------ backward
// x_seq (TIN); every gradient, the initial potential and grad_x_seq [T,N], grad_v_init [N] in TG; PLIF: block partial sums of
// dL/dr go to partial[gridDim.x], the last block to finish (ticket counter) adds them
// in index order into grad_r[0] — a deterministic single-launch reduction.
// LEAN: T is a multiple of TC, scalar initial potential, no gradient flowing in through v_last or v_seq.
template <typename TIN, typename TG, int V, int TC, int KIND, bool LEAN = false>
__global__ void __launch_bounds__(256, 2)
scan_backward_kernel(ScanParams p, const TIN* __restrict__ x_seq, const TG* __restrict__ grad_spike_seq,
                     const TG* __restrict__ grad_v_last, const TG* __restrict__ grad_v_seq,
                     const float* __restrict__ ckpt, TG* __restrict__ grad_x_seq, TG* __restrict__ grad_v_init,
                     float* __restrict__ grad_r, float* __restrict__ partial, unsigned int* __restrict__ ticket) {
    const long long gtid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long n0 = gtid * V;
    constexpr bool plif = Neuron<KIND>::kPlif;
    if constexpr (LEAN) {
        p.v_init = nullptr; grad_v_last = nullptr; grad_v_seq = nullptr;
        if constexpr (!plif) { if (n0 >= p.N) return; }     // the PLIF block reduction needs every thread
    }
    const bool active = (LEAN && !plif) ? true : (n0 < p.N);
    const Neuron<KIND> nrn(p);
    constexpr bool need_v = Neuron<KIND>::kNeedsV;
    const float dhdx = nrn.dh_dx();
    const float dhdv_const = nrn.dh_dv(0.0f);   // used when dh/dv does not depend on v
    const float kd = p.detach_reset ? 0.0f : 1.0f;
    const float k_s = p.soft_reset ? 0.0f : 1.0f;
    const float k_a = kd * (p.soft_reset ? -p.v_th : p.v_reset);
    const float k_b = kd * (p.soft_reset ? 0.0f : -1.0f);

    float c[V];     // dL/dv_t flowing in from step t+1
    float gr = 0.0f;
    if (active && grad_v_last != nullptr) {
        load_vec<TG, V>(grad_v_last + n0, c);
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
            load_vec<TG, V>(reinterpret_cast<const TG*>(p.v_init) + n0, v0);
        } else {
#pragma unroll
            for (int j = 0; j < V; ++j) v0[j] = p.v_init_scalar;
        }
        // issue every load of the chunk (inputs and upstream gradients) before any use
        Pack<TIN, V> xr[TC];
        Pack<TG, V> gr_raw[TC];
#pragma unroll
        for (int i = 0; i < TC; ++i) {
            if (active && (LEAN || t0 + i < p.T)) {
                xr[i] = load_raw_stream<TIN, V>(x_seq + (long long)(t0 + i) * p.N + n0);
                gr_raw[i] = load_raw_stream<TG, V>(grad_spike_seq + (long long)(t0 + i) * p.N + n0);
            }
        }
        // recompute the membrane trajectory of the chunk
        float h[TC][V];
        {
            float v[V];
#pragma unroll
            for (int j = 0; j < V; ++j) v[j] = v0[j];
#pragma unroll
            for (int i = 0; i < TC; ++i) {
                if (LEAN || t0 + i < p.T) {
                    float x[V];
                    unpack<TIN, V>(xr[i], x);
#pragma unroll
                    for (int j = 0; j < V; ++j) {
                        const float hh = nrn.charge(x[j], v[j]);
                        h[i][j] = hh;
                        v[j] = nrn.reset(hh, nrn.fire(hh));
                    }
                }
            }
        }
        // reverse walk.  d v_t / d h_t = 1 - k_s s + sg (k_a + k_b h) with uniform constants:
        //   soft reset: k_s = 0, k_a = -v_th, k_b = 0;  hard: k_s = 1, k_a = v_reset, k_b = -1;
        //   detach_reset zeroes k_a and k_b.
#pragma unroll
        for (int i = TC - 1; i >= 0; --i) {
            if (LEAN || t0 + i < p.T) {
                const long long off = (long long)(t0 + i) * p.N + n0;
                float gs[V], gv[V], gx[V], sg[V];
                if (active) {
                    unpack<TG, V>(gr_raw[i], gs);
                    if (grad_v_seq != nullptr) load_vec_stream<TG, V>(grad_v_seq + off, gv);
                } else {
#pragma unroll
                    for (int j = 0; j < V; ++j) gs[j] = 0.0f;
                }
#pragma unroll
                for (int j = 0; j < V; ++j) sg[j] = h[i][j] - p.v_th;
                surrogate_grad_vec<V>(p.sg_id, sg, p.sg_p0, p.sg_p1);   // one switch per V elements
#pragma unroll
                for (int j = 0; j < V; ++j) {
                    const float hh = h[i][j];
                    const float s = nrn.fire(hh) ? 1.0f : 0.0f;
                    const float g = c[j] + ((active && grad_v_seq != nullptr) ? gv[j] : 0.0f);
                    const float dv_dh = fmaf(sg[j], fmaf(k_b, hh, k_a), fmaf(-k_s, s, 1.0f));
                    const float gh = fmaf(gs[j], sg[j], g * dv_dh);
                    if constexpr (need_v) {
                        float vprev;
                        if (i == 0) vprev = v0[j];
                        else { const float hp = h[i > 0 ? i - 1 : 0][j]; vprev = nrn.reset(hp, nrn.fire(hp)); }
                        if constexpr (plif) gr += (KIND == NK_PLIF_DI) ? gh * (hh - vprev) * nrn.inv_r : gh * (nrn.vr - vprev);
                        c[j] = gh * nrn.dh_dv(vprev);
                    } else {
                        c[j] = gh * dhdv_const;
                    }
                    gx[j] = gh * dhdx;
                }
                if (active) store_vec<TG, V>(grad_x_seq + off, gx);
            }
        }
    }
    if (active && grad_v_init != nullptr) store_vec<TG, V>(grad_v_init + n0, c);

    if constexpr (plif) {
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
