// Host launchers and torch bindings for the neuron scan kernels.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <cuda_fp8.h>

#include "neuron_scan_launch.cuh"

namespace sjb200 {
namespace {

constexpr int kThreads = 256;

template <typename T>
bool aligned(const void* p, int v) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) % (sizeof(T) * v)) == 0; }

struct Dims { int T; long long N; };

Dims seq_dims(const at::Tensor& x_seq) {
    TORCH_CHECK(x_seq.dim() >= 1, "x_seq must have a leading time axis");
    Dims d;
    d.T = (int)x_seq.size(0);
    d.N = d.T > 0 ? x_seq.numel() / d.T : 0;
    return d;
}

ScanParams make_params(const Dims& d, int64_t kind, double tau, double q0, double q1, double q2,
                       const c10::optional<at::Tensor>& r, double v_th, double v_reset, bool soft_reset,
                       const c10::optional<at::Tensor>& v_init, double v_init_scalar) {
    ScanParams p{};
    p.T = d.T; p.N = d.N; p.kind = (int)kind;
    p.inv_tau = 1.0f / (float)tau; p.q0 = (float)q0; p.q1 = (float)q1; p.q2 = (float)q2;
    p.r_ptr = nullptr;
    if (kind == NK_PLIF_DI || kind == NK_PLIF_NDI) {
        TORCH_CHECK(r.has_value() && r->is_cuda() && r->scalar_type() == at::kFloat && r->numel() == 1,
                    "PLIF needs r = sigmoid(w) as a one-element fp32 CUDA tensor");
        p.r_ptr = r->data_ptr<float>();
    }
    p.v_th = (float)v_th; p.v_reset = (float)v_reset; p.soft_reset = soft_reset ? 1 : 0;
    p.v_init = (v_init.has_value() && v_init->defined() && v_init->numel() > 0) ? v_init->data_ptr() : nullptr;
    p.v_init_scalar = (float)v_init_scalar;
    return p;
}

// scalar_t: storage type of x_seq; state_t: type of spikes, potentials and gradients (bf16 when x is stored as fp8, e4m3 or
// e5m2).  The recurrence itself always runs in fp32 registers, whatever the storage types.
#define SJ_DISPATCH_FLOATING(DTYPE, ...)                                                                      \
    switch (DTYPE) {                                                                                           \
    case at::kFloat: { using scalar_t = float; using state_t = float; __VA_ARGS__; break; }                    \
    case at::kHalf: { using scalar_t = __half; using state_t = __half; __VA_ARGS__; break; }                   \
    case at::kBFloat16: { using scalar_t = __nv_bfloat16; using state_t = __nv_bfloat16; __VA_ARGS__; break; } \
    case at::kFloat8_e4m3fn: { using scalar_t = __nv_fp8_e4m3; using state_t = __nv_bfloat16; __VA_ARGS__; break; } \
    case at::kFloat8_e5m2: { using scalar_t = __nv_fp8_e5m2; using state_t = __nv_bfloat16; __VA_ARGS__; break; }   \
    default: TORCH_CHECK(false, "neuron scan: unsupported dtype ", DTYPE);                                     \
    }

at::ScalarType state_dtype(at::ScalarType x) { return (x == at::kFloat8_e4m3fn || x == at::kFloat8_e5m2) ? at::kBFloat16 : x; }

int chunk_for(int T) { return T <= 4 ? 4 : 8; }

}  // namespace

int64_t scan_chunk(int64_t T) { return chunk_for((int)T); }

// returns (spike_seq, v_last, v_seq | empty, packed | empty, ckpt | empty)
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor> scan_forward(
    const at::Tensor& x_seq, const c10::optional<at::Tensor>& v_init, double v_init_scalar,
    const c10::optional<at::Tensor>& r, int64_t kind, double tau, double q0, double q1, double q2, double v_th,
    double v_reset, bool soft_reset, bool store_v_seq, bool pack_bits, bool save_ckpt, bool bits_only) {
    TORCH_CHECK(x_seq.is_cuda(), "scan_forward: x_seq must be a CUDA tensor");
    TORCH_CHECK(!bits_only || pack_bits, "scan_forward: bits_only needs pack_bits");
    const c10::cuda::CUDAGuard guard(x_seq.device());
    at::Tensor x = x_seq.contiguous();
    const Dims d = seq_dims(x);
    c10::optional<at::Tensor> vi;
    if (v_init.has_value() && v_init->defined() && v_init->numel() > 0) {
        TORCH_CHECK(v_init->numel() == d.N, "v_init must have one value per neuron");
        vi = v_init->to(state_dtype(x.scalar_type())).contiguous();
    }
    const ScanParams p = make_params(d, kind, tau, q0, q1, q2, r, v_th, v_reset, soft_reset, vi, v_init_scalar);

    const auto sopt = x.options().dtype(state_dtype(x.scalar_type()));
    // bits_only: the spikes leave the kernel as 1 bit per neuron and nothing else (the dense tensor has no elements)
    at::Tensor spike = bits_only ? at::empty({0}, sopt) : at::empty(x.sizes(), sopt);
    std::vector<int64_t> state_shape(x.sizes().begin() + 1, x.sizes().end());
    at::Tensor v_last = at::empty(state_shape, sopt);
    // a zero-element tensor stands for an absent optional output (each output gets its own)
    auto none = [&]() { return at::empty({0}, x.options()); };
    c10::optional<at::Tensor> v_seq, packed, ckpt;
    if (store_v_seq) v_seq = at::empty(x.sizes(), sopt);
    if (pack_bits) packed = at::empty({d.T, (d.N + 31) / 32}, x.options().dtype(at::kInt));
    const int TC = chunk_for(d.T);
    const int n_ckpt = (d.T + TC - 1) / TC - 1;
    if (save_ckpt && n_ckpt > 0) ckpt = at::empty({n_ckpt, d.N}, x.options().dtype(at::kFloat));
    if (d.N == 0 || d.T == 0) {
        return {spike, v_last, v_seq.has_value() ? *v_seq : none(), packed.has_value() ? *packed : none(), ckpt.has_value() ? *ckpt : none()};
    }
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    SJ_DISPATCH_FLOATING(x.scalar_type(), {
        constexpr int VV = 16 / sizeof(state_t);
        const bool vec = (d.N % VV == 0) && aligned<scalar_t>(x.data_ptr(), VV) && (bits_only || aligned<state_t>(spike.data_ptr(), VV)) &&
                         aligned<state_t>(v_last.data_ptr(), VV) && aligned<state_t>(p.v_init, VV) &&
                         (!v_seq.has_value() || aligned<state_t>(v_seq->data_ptr(), VV)) &&
                         (!ckpt.has_value() || aligned<float>(ckpt->data_ptr(), VV));
        const int V = vec ? (TC == 8 ? 4 : VV) : 1;
        const long long threads_needed = (d.N + V - 1) / V;
        const unsigned grid = (unsigned)((threads_needed + kThreads - 1) / kThreads);
        ScanFwdPtrs io{x.data_ptr(), bits_only ? nullptr : spike.data_ptr(), v_last.data_ptr(),
                       v_seq.has_value() ? v_seq->data_ptr() : nullptr,
                       packed.has_value() ? reinterpret_cast<uint32_t*>(packed->data_ptr()) : nullptr,
                       ckpt.has_value() ? ckpt->data_ptr<float>() : nullptr};
        scan_forward_launch<scalar_t, state_t>(p, io, vec, TC, grid, stream);
    });
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return {spike, v_last, v_seq.has_value() ? *v_seq : none(), packed.has_value() ? *packed : none(), ckpt.has_value() ? *ckpt : none()};
}

// returns (grad_x_seq, grad_v_init | empty, grad_r | empty)
// `scratch` (PLIF only): fp32 tensor with at least grid+1 elements whose LAST element is an
// always-zero-between-launches ticket counter; the kernel restores it to zero.
std::tuple<at::Tensor, at::Tensor, at::Tensor> scan_backward(
    const at::Tensor& grad_spike_seq, const c10::optional<at::Tensor>& grad_v_last,
    const c10::optional<at::Tensor>& grad_v_seq, const at::Tensor& x_seq, const c10::optional<at::Tensor>& v_init,
    double v_init_scalar, const c10::optional<at::Tensor>& r, const c10::optional<at::Tensor>& ckpt, int64_t kind,
    double tau, double q0, double q1, double q2, double v_th, double v_reset, bool soft_reset, int64_t sg_id,
    double sg_p0, double sg_p1, bool detach_reset, bool need_grad_v_init) {
    TORCH_CHECK(x_seq.is_cuda(), "scan_backward: x_seq must be a CUDA tensor");
    const c10::cuda::CUDAGuard guard(x_seq.device());
    at::Tensor x = x_seq.contiguous();
    const Dims d = seq_dims(x);
    const at::ScalarType sdt = state_dtype(x.scalar_type());
    at::Tensor gs = grad_spike_seq.to(sdt).contiguous();
    TORCH_CHECK(gs.numel() == x.numel(), "grad_spike_seq must match x_seq");
    c10::optional<at::Tensor> vi, gvl, gvs;
    if (v_init.has_value() && v_init->defined() && v_init->numel() > 0) vi = v_init->to(sdt).contiguous();
    if (grad_v_last.has_value() && grad_v_last->defined() && grad_v_last->numel() > 0)
        gvl = grad_v_last->to(sdt).contiguous();
    if (grad_v_seq.has_value() && grad_v_seq->defined() && grad_v_seq->numel() > 0)
        gvs = grad_v_seq->to(sdt).contiguous();
    ScanParams p = make_params(d, kind, tau, q0, q1, q2, r, v_th, v_reset, soft_reset, vi, v_init_scalar);
    p.sg_id = (int)sg_id; p.sg_p0 = (float)sg_p0; p.sg_p1 = (float)sg_p1; p.detach_reset = detach_reset ? 1 : 0;

    const int TC = chunk_for(d.T);
    const int n_ckpt = (d.T + TC - 1) / TC - 1;
    const float* ckpt_ptr = nullptr;
    if (n_ckpt > 0) {
        TORCH_CHECK(ckpt.has_value() && ckpt->defined() && ckpt->numel() == (int64_t)n_ckpt * d.N,
                    "scan_backward: T > chunk needs the forward checkpoints");
        ckpt_ptr = ckpt->data_ptr<float>();
    }
    const auto sopt = x.options().dtype(sdt);
    at::Tensor gx = at::empty(x.sizes(), sopt);
    std::vector<int64_t> state_shape(x.sizes().begin() + 1, x.sizes().end());
    at::Tensor gvi = need_grad_v_init ? at::empty(state_shape, sopt) : at::empty({0}, sopt);
    const bool plif = (kind == NK_PLIF_DI || kind == NK_PLIF_NDI);
    at::Tensor grad_r = plif ? at::zeros({1}, x.options().dtype(at::kFloat)) : at::empty({0}, x.options());
    if (d.N == 0 || d.T == 0) return {gx, gvi, grad_r};

    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    SJ_DISPATCH_FLOATING(x.scalar_type(), {
        constexpr int VV = 16 / sizeof(state_t);
        const bool vec = (d.N % VV == 0) && aligned<scalar_t>(x.data_ptr(), VV) && aligned<state_t>(gs.data_ptr(), VV) &&
                         aligned<state_t>(gx.data_ptr(), VV) && aligned<state_t>(p.v_init, VV) &&
                         (!gvl.has_value() || aligned<state_t>(gvl->data_ptr(), VV)) &&
                         (!gvs.has_value() || aligned<state_t>(gvs->data_ptr(), VV)) &&
                         (!need_grad_v_init || aligned<state_t>(gvi.data_ptr(), VV)) && aligned<float>(ckpt_ptr, VV);
        const int V = vec ? (TC == 8 ? 4 : VV) : 1;
        const long long threads_needed = (d.N + V - 1) / V;
        const unsigned grid = (unsigned)((threads_needed + kThreads - 1) / kThreads);
        at::Tensor scratch;
        float* partial = nullptr;
        unsigned int* ticket = nullptr;
        if (plif) {  // block partials + ticket (zeroed once; the kernel leaves the ticket at zero)
            scratch = at::zeros({(int64_t)grid + 1}, x.options().dtype(at::kFloat));
            partial = scratch.data_ptr<float>();
            ticket = reinterpret_cast<unsigned int*>(partial + grid);
        }
        const void* gvl_p = gvl.has_value() ? gvl->data_ptr() : nullptr;
        const void* gvs_p = gvs.has_value() ? gvs->data_ptr() : nullptr;
        void* gvi_p = need_grad_v_init ? gvi.data_ptr() : nullptr;
        float* gr_p = plif ? grad_r.data_ptr<float>() : nullptr;
        ScanBwdPtrs io{x.data_ptr(), gs.data_ptr(), gvl_p, gvs_p, ckpt_ptr, gx.data_ptr(), gvi_p, gr_p, partial, ticket};
        scan_backward_launch<scalar_t, state_t>(p, io, vec, TC, grid, stream);
    });
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return {gx, gvi, grad_r};
}

}  // namespace sjb200

TORCH_LIBRARY_FRAGMENT(sjb200, m) {
    m.def("scan_chunk(int T) -> int", &sjb200::scan_chunk);
    m.def("scan_forward(Tensor x_seq, Tensor? v_init, float v_init_scalar, Tensor? r, int kind, float tau, float q0, "
          "float q1, float q2, float v_th, float v_reset, bool soft_reset, bool store_v_seq, bool pack_bits, "
          "bool save_ckpt, bool bits_only=False) -> (Tensor, Tensor, Tensor, Tensor, Tensor)");
    m.def("scan_backward(Tensor grad_spike_seq, Tensor? grad_v_last, Tensor? grad_v_seq, Tensor x_seq, Tensor? v_init, "
          "float v_init_scalar, Tensor? r, Tensor? ckpt, int kind, float tau, float q0, float q1, float q2, float v_th, "
          "float v_reset, bool soft_reset, int sg_id, float sg_p0, float sg_p1, bool detach_reset, "
          "bool need_grad_v_init) -> (Tensor, Tensor, Tensor)");
}

TORCH_LIBRARY_IMPL(sjb200, CUDA, m) {
    m.impl("scan_forward", &sjb200::scan_forward);
    m.impl("scan_backward", &sjb200::scan_backward);
}
