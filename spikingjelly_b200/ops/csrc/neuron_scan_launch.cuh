// Type-erased launch interface of the neuron scan kernels.  One translation unit per
// storage dtype instantiates the kernels (neuron_scan_inst_*.cu) so that they compile in
// parallel; neuron_scan.cu holds the dtype-independent host logic and the bindings.
#pragma once
#include "neuron_scan.cuh"

namespace sjb200 {

struct ScanFwdPtrs {
    const void* x_seq; void* spike_seq; void* v_last; void* v_seq; uint32_t* packed; float* ckpt;
};
struct ScanBwdPtrs {
    const void* x_seq; const void* grad_spike_seq; const void* grad_v_last; const void* grad_v_seq; const float* ckpt;
    void* grad_x_seq; void* grad_v_init; float* grad_r; float* partial; unsigned int* ticket;
};

// `vec`: use vector accesses (caller checked divisibility and alignment for 16 bytes); TC: chunk
// (4 or 8 steps).  Chunks of 8 steps use 4 elements per thread whatever the dtype, so that the
// recomputed trajectory (TC x V floats) stays in registers.
template <typename T, typename TO = T> void scan_forward_launch(const ScanParams& p, const ScanFwdPtrs& io, bool vec, int TC, unsigned grid, cudaStream_t s);
template <typename T, typename TO = T> void scan_backward_launch(const ScanParams& p, const ScanBwdPtrs& io, bool vec, int TC, unsigned grid, cudaStream_t s);

// (the instantiation macro below names its type parameter T, so p.T cannot be spelled inside it)
inline int scan_steps(const ScanParams& p) { return p.T; }

#define SJ_SCAN_KIND_SWITCH(KIND_VALUE, ...)                                           \
    switch (KIND_VALUE) {                                                              \
    case NK_IF: { constexpr int KIND = NK_IF; __VA_ARGS__; break; }                    \
    case NK_LIF_DI: { constexpr int KIND = NK_LIF_DI; __VA_ARGS__; break; }            \
    case NK_LIF_NDI: { constexpr int KIND = NK_LIF_NDI; __VA_ARGS__; break; }          \
    case NK_PLIF_DI: { constexpr int KIND = NK_PLIF_DI; __VA_ARGS__; break; }          \
    case NK_PLIF_NDI: { constexpr int KIND = NK_PLIF_NDI; __VA_ARGS__; break; }        \
    case NK_QIF: { constexpr int KIND = NK_QIF; __VA_ARGS__; break; }                  \
    default: { constexpr int KIND = NK_EIF; __VA_ARGS__; break; }                      \
    }

#define SJ_SCAN_INSTANTIATE(T)                                                                                      \
    template <>                                                                                                     \
    void scan_forward_launch<T>(const ScanParams& p, const ScanFwdPtrs& io, bool vec, int TC, unsigned grid,       \
                                cudaStream_t s) {                                                                   \
        constexpr int VV = 16 / sizeof(T);                                                                          \
        constexpr int V8 = 4;                                                                                       \
        auto x = reinterpret_cast<const T*>(io.x_seq);                                                              \
        auto sp = reinterpret_cast<T*>(io.spike_seq);                                                               \
        auto vl = reinterpret_cast<T*>(io.v_last);                                                                  \
        auto vs = reinterpret_cast<T*>(io.v_seq);                                                                   \
        const bool lean = vec && scan_steps(p) % TC == 0 && p.v_init == nullptr && io.v_seq == nullptr && io.packed == nullptr;   \
        SJ_SCAN_KIND_SWITCH(p.kind, {                                                                               \
            if (lean && TC == 4) scan_forward_kernel<T, T, VV, 4, KIND, true><<<grid, 256, 0, s>>>(p, x, sp, vl, vs, io.packed, io.ckpt); \
            else if (lean) scan_forward_kernel<T, T, V8, 8, KIND, true><<<grid, 256, 0, s>>>(p, x, sp, vl, vs, io.packed, io.ckpt);       \
            else if (vec && TC == 4) scan_forward_kernel<T, T, VV, 4, KIND><<<grid, 256, 0, s>>>(p, x, sp, vl, vs, io.packed, io.ckpt); \
            else if (vec) scan_forward_kernel<T, T, V8, 8, KIND><<<grid, 256, 0, s>>>(p, x, sp, vl, vs, io.packed, io.ckpt);       \
            else if (TC == 4) scan_forward_kernel<T, T, 1, 4, KIND><<<grid, 256, 0, s>>>(p, x, sp, vl, vs, io.packed, io.ckpt);    \
            else scan_forward_kernel<T, T, 1, 8, KIND><<<grid, 256, 0, s>>>(p, x, sp, vl, vs, io.packed, io.ckpt);                 \
        });                                                                                                         \
    }                                                                                                               \
    template <>                                                                                                     \
    void scan_backward_launch<T>(const ScanParams& p, const ScanBwdPtrs& io, bool vec, int TC, unsigned grid,      \
                                 cudaStream_t s) {                                                                  \
        constexpr int VV = 16 / sizeof(T);                                                                          \
        constexpr int V8 = 4;                                                                                       \
        auto x = reinterpret_cast<const T*>(io.x_seq);                                                              \
        auto gs = reinterpret_cast<const T*>(io.grad_spike_seq);                                                    \
        auto gvl = reinterpret_cast<const T*>(io.grad_v_last);                                                      \
        auto gvs = reinterpret_cast<const T*>(io.grad_v_seq);                                                       \
        auto gx = reinterpret_cast<T*>(io.grad_x_seq);                                                              \
        auto gvi = reinterpret_cast<T*>(io.grad_v_init);                                                            \
        const bool lean = vec && scan_steps(p) % TC == 0 && p.v_init == nullptr && io.grad_v_last == nullptr && io.grad_v_seq == nullptr; \
        SJ_SCAN_KIND_SWITCH(p.kind, {                                                                               \
            if (lean && TC == 4) scan_backward_kernel<T, T, VV, 4, KIND, true><<<grid, 256, 0, s>>>(p, x, gs, gvl, gvs, io.ckpt, gx, gvi, io.grad_r, io.partial, io.ticket); \
            else if (lean) scan_backward_kernel<T, T, V8, 8, KIND, true><<<grid, 256, 0, s>>>(p, x, gs, gvl, gvs, io.ckpt, gx, gvi, io.grad_r, io.partial, io.ticket);       \
            else if (vec && TC == 4) scan_backward_kernel<T, T, VV, 4, KIND><<<grid, 256, 0, s>>>(p, x, gs, gvl, gvs, io.ckpt, gx, gvi, io.grad_r, io.partial, io.ticket); \
            else if (vec) scan_backward_kernel<T, T, V8, 8, KIND><<<grid, 256, 0, s>>>(p, x, gs, gvl, gvs, io.ckpt, gx, gvi, io.grad_r, io.partial, io.ticket);       \
            else if (TC == 4) scan_backward_kernel<T, T, 1, 4, KIND><<<grid, 256, 0, s>>>(p, x, gs, gvl, gvs, io.ckpt, gx, gvi, io.grad_r, io.partial, io.ticket);    \
            else scan_backward_kernel<T, T, 1, 8, KIND><<<grid, 256, 0, s>>>(p, x, gs, gvl, gvs, io.ckpt, gx, gvi, io.grad_r, io.partial, io.ticket);                 \
        });                                                                                                         \
    }

#define SJ_SCAN_INSTANTIATE2(T, TO)                                                                                      \
    template <>                                                                                                     \
    void scan_forward_launch<T, TO>(const ScanParams& p, const ScanFwdPtrs& io, bool vec, int TC, unsigned grid,       \
                                cudaStream_t s) {                                                                   \
        constexpr int VV = 16 / sizeof(TO);                                                                          \
        constexpr int V8 = 4;                                                                                       \
        auto x = reinterpret_cast<const T*>(io.x_seq);                                                              \
        auto sp = reinterpret_cast<TO*>(io.spike_seq);                                                               \
        auto vl = reinterpret_cast<TO*>(io.v_last);                                                                  \
        auto vs = reinterpret_cast<TO*>(io.v_seq);                                                                   \
        const bool lean = vec && scan_steps(p) % TC == 0 && p.v_init == nullptr && io.v_seq == nullptr && io.packed == nullptr;   \
        SJ_SCAN_KIND_SWITCH(p.kind, {                                                                               \
            if (lean && TC == 4) scan_forward_kernel<T, TO, VV, 4, KIND, true><<<grid, 256, 0, s>>>(p, x, sp, vl, vs, io.packed, io.ckpt); \
            else if (lean) scan_forward_kernel<T, TO, V8, 8, KIND, true><<<grid, 256, 0, s>>>(p, x, sp, vl, vs, io.packed, io.ckpt);       \
            else if (vec && TC == 4) scan_forward_kernel<T, TO, VV, 4, KIND><<<grid, 256, 0, s>>>(p, x, sp, vl, vs, io.packed, io.ckpt); \
            else if (vec) scan_forward_kernel<T, TO, V8, 8, KIND><<<grid, 256, 0, s>>>(p, x, sp, vl, vs, io.packed, io.ckpt);       \
            else if (TC == 4) scan_forward_kernel<T, TO, 1, 4, KIND><<<grid, 256, 0, s>>>(p, x, sp, vl, vs, io.packed, io.ckpt);    \
            else scan_forward_kernel<T, TO, 1, 8, KIND><<<grid, 256, 0, s>>>(p, x, sp, vl, vs, io.packed, io.ckpt);                 \
        });                                                                                                         \
    }                                                                                                               \
    template <>                                                                                                     \
    void scan_backward_launch<T, TO>(const ScanParams& p, const ScanBwdPtrs& io, bool vec, int TC, unsigned grid,      \
                                 cudaStream_t s) {                                                                  \
        constexpr int VV = 16 / sizeof(TO);                                                                          \
        constexpr int V8 = 4;                                                                                       \
        auto x = reinterpret_cast<const T*>(io.x_seq);                                                              \
        auto gs = reinterpret_cast<const TO*>(io.grad_spike_seq);                                                    \
        auto gvl = reinterpret_cast<const TO*>(io.grad_v_last);                                                      \
        auto gvs = reinterpret_cast<const TO*>(io.grad_v_seq);                                                       \
        auto gx = reinterpret_cast<TO*>(io.grad_x_seq);                                                              \
        auto gvi = reinterpret_cast<TO*>(io.grad_v_init);                                                            \
        const bool lean = vec && scan_steps(p) % TC == 0 && p.v_init == nullptr && io.grad_v_last == nullptr && io.grad_v_seq == nullptr; \
        SJ_SCAN_KIND_SWITCH(p.kind, {                                                                               \
            if (lean && TC == 4) scan_backward_kernel<T, TO, VV, 4, KIND, true><<<grid, 256, 0, s>>>(p, x, gs, gvl, gvs, io.ckpt, gx, gvi, io.grad_r, io.partial, io.ticket); \
            else if (lean) scan_backward_kernel<T, TO, V8, 8, KIND, true><<<grid, 256, 0, s>>>(p, x, gs, gvl, gvs, io.ckpt, gx, gvi, io.grad_r, io.partial, io.ticket);       \
            else if (vec && TC == 4) scan_backward_kernel<T, TO, VV, 4, KIND><<<grid, 256, 0, s>>>(p, x, gs, gvl, gvs, io.ckpt, gx, gvi, io.grad_r, io.partial, io.ticket); \
            else if (vec) scan_backward_kernel<T, TO, V8, 8, KIND><<<grid, 256, 0, s>>>(p, x, gs, gvl, gvs, io.ckpt, gx, gvi, io.grad_r, io.partial, io.ticket);       \
            else if (TC == 4) scan_backward_kernel<T, TO, 1, 4, KIND><<<grid, 256, 0, s>>>(p, x, gs, gvl, gvs, io.ckpt, gx, gvi, io.grad_r, io.partial, io.ticket);    \
            else scan_backward_kernel<T, TO, 1, 8, KIND><<<grid, 256, 0, s>>>(p, x, gs, gvl, gvs, io.ckpt, gx, gvi, io.grad_r, io.partial, io.ticket);                 \
        });                                                                                                         \
    }


}  // namespace sjb200
