"""Shape-and-dtype ("fake" / meta) implementations of the native operators, so that models which call them can be traced
by ``torch.export`` / ``torch.compile`` / ``make_fx`` and inspected with fake tensors.  Registered once, right after the
library is loaded (role of the fake registrations in ``triton_kernel/flexsn/custom_ops.py:593-1118`` and
``cuda_kernel/auto_cuda/*`` custom-op migration in the reference)."""
from __future__ import annotations

import torch

_done = False


def register() -> None:
    global _done
    if _done:
        return
    _done = True
    reg = torch.library.register_fake

    @reg("sjb200::gemm_16bit")
    def _(a, b, a_mn, b_mn, out_f32, split_k):
        M = a.shape[1] if a_mn else a.shape[0]
        N = b.shape[1] if b_mn else b.shape[0]
        return a.new_empty((M, N), dtype=torch.float32 if out_f32 else a.dtype)

    @reg("sjb200::gemm_16bit_stats")
    def _(a, b, a_mn, b_mn):
        M = a.shape[1] if a_mn else a.shape[0]
        N = b.shape[1] if b_mn else b.shape[0]
        K = a.shape[0] if a_mn else a.shape[1]
        pair = M >= 256 and N >= 256 and (K + 63) // 64 >= 16       # the shapes that run on the two-CTA kernel (256-row tiles)
        rows = (M + 255) // 256 * 8 if pair else (M + 127) // 128 * 4
        return a.new_empty((M, N)), a.new_empty((rows, 2, N), dtype=torch.float32)

    @reg("sjb200::maxpool3x3s2_nhwc_forward")
    def _(x):
        n, h, w, c = x.shape
        shape = (n, (h - 1) // 2 + 1, (w - 1) // 2 + 1, c)
        return x.new_empty(shape), x.new_empty(shape, dtype=torch.uint8)

    @reg("sjb200::maxpool3x3s2_nhwc_backward")
    def _(g_out, idx, H, W):
        return g_out.new_empty((g_out.shape[0], H, W, g_out.shape[3]))

    @reg("sjb200::im2col_nhwc")
    def _(x, KH, KW, sh, sw, ph, pw):
        n, h, w, c = x.shape
        oh, ow = (h + 2 * ph - KH) // sh + 1, (w + 2 * pw - KW) // sw + 1
        return x.new_empty((n * oh * ow, (KH * KW * c + 7) // 8 * 8))

    @reg("sjb200::rope_qkv_forward")
    def _(qkv, cos, sin, offset):
        n, s_, h, _, d = qkv.shape
        return tuple(qkv.new_empty((n, s_, h, d)) for _ in range(3))

    @reg("sjb200::rope_qkv_backward")
    def _(gq, gk, gv, cos, sin, offset):
        n, s_, h, d = gq.shape
        return gq.new_empty((n, s_, h, 3, d))

    @reg("sjb200::gemm_fp8")
    def _(a, b, alpha, out_f32, split_k, alpha2=None, bias=None):
        return a.new_empty((a.shape[0], b.shape[0]), dtype=torch.float32 if out_f32 else torch.bfloat16)

    @reg("sjb200::fp8_quantize")
    def _(x, e5m2):
        return x.new_empty(x.shape, dtype=torch.float8_e5m2 if e5m2 else torch.float8_e4m3fn), x.new_empty((1,), dtype=torch.float32)

    @reg("sjb200::fp8_quantize_delayed")
    def _(x, amax3, slot, e5m2):
        return x.new_empty(x.shape, dtype=torch.float8_e5m2 if e5m2 else torch.float8_e4m3fn), x.new_empty((1,), dtype=torch.float32)

    @reg("sjb200::fp8_quantize_transpose")
    def _(x, amax3, slot, e5m2):
        f8 = torch.float8_e5m2 if e5m2 else torch.float8_e4m3fn
        return x.new_empty(x.shape, dtype=f8), x.new_empty((x.shape[1], x.shape[0]), dtype=f8), x.new_empty((1,), dtype=torch.float32)

    @reg("sjb200::psn_forward")
    def _(x, w, b):
        return torch.empty_like(x)

    @reg("sjb200::psn_backward")
    def _(x, grad_s, w, b, surrogate_id, p0, p1):
        return torch.empty_like(x), torch.empty_like(x)

    @reg("sjb200::psn_backward_small")
    def _(x, grad_s, w, b, surrogate_id, p0, p1):
        T = x.shape[0]
        return torch.empty_like(x), x.new_empty((T, T), dtype=torch.float32), x.new_empty((T,), dtype=torch.float32)

    @reg("sjb200::bit_pack")
    def _(x):
        return x.new_empty(((x.numel() + 7) // 8,), dtype=torch.uint8)

    @reg("sjb200::bit_unpack")
    def _(packed, n, dtype):
        return packed.new_empty((n,), dtype=dtype)

    @reg("sjb200::ssa_forward")
    def _(S, L, H, scale):
        return S.new_empty((*S.shape[:-1], S.shape[-1] // 3))

    @reg("sjb200::ssa_backward")
    def _(dO, S, L, H, scale):
        return torch.empty_like(S)

    # ------------------------------------------------------------------ neuron scan
    def _state_dtype(x):
        return torch.bfloat16 if x.dtype in (torch.float8_e4m3fn, torch.float8_e5m2) else x.dtype

    @reg("sjb200::scan_forward")
    def _(x_seq, v_init, v_init_scalar, r, kind, tau, q0, q1, q2, v_th, v_reset, soft_reset, store_v_seq, pack_bits, save_ckpt,
          bits_only=False):
        sd = _state_dtype(x_seq)
        T = x_seq.shape[0]
        N = x_seq.numel() // T if T else 0
        chunk = 4 if T <= 4 else 8
        n_ckpt = (T + chunk - 1) // chunk - 1
        none = lambda: x_seq.new_empty((0,))
        return (x_seq.new_empty((0,) if bits_only else x_seq.shape, dtype=sd), x_seq.new_empty(x_seq.shape[1:], dtype=sd),
                x_seq.new_empty(x_seq.shape, dtype=sd) if store_v_seq else none(),
                x_seq.new_empty((T, (N + 31) // 32), dtype=torch.int32) if pack_bits else none(),
                x_seq.new_empty((n_ckpt, N), dtype=torch.float32) if (save_ckpt and n_ckpt > 0) else none())

    @reg("sjb200::scan_backward")
    def _(grad_spike_seq, grad_v_last, grad_v_seq, x_seq, v_init, v_init_scalar, r, ckpt, kind, tau, q0, q1, q2, v_th, v_reset,
          soft_reset, sg_id, sg_p0, sg_p1, detach_reset, need_grad_v_init):
        sd = _state_dtype(x_seq)
        gvi = x_seq.new_empty(x_seq.shape[1:], dtype=sd) if need_grad_v_init else x_seq.new_empty((0,), dtype=sd)
        grad_r = x_seq.new_empty((1,), dtype=torch.float32) if r is not None else x_seq.new_empty((0,))
        return x_seq.new_empty(x_seq.shape, dtype=sd), gvi, grad_r

    # ------------------------------------------------------------------ batch norm + neuron
    def _bn_four(like, C):
        return tuple(like.new_empty((C,), dtype=torch.float32) for _ in range(4))

    @reg("sjb200::bn_coefficients")
    def _(y, gamma, beta, running_mean, running_var, training, momentum, eps):
        return _bn_four(y, y.shape[-1])

    @reg("sjb200::bn_coefficients_partial")
    def _(partial, rows, gamma, beta, running_mean, running_var, momentum, eps):
        return _bn_four(partial, partial.shape[-1])

    @reg("sjb200::bn_lif_forward")
    def _(y, scale, shift, residual, kind, tau, v_th, v_reset, soft_reset, v_init, save_ckpt):
        T = y.shape[0]
        n_ckpt = (T + 3) // 4 - 1
        ckpt = y.new_empty((n_ckpt, y.numel() // T), dtype=torch.float32) if (save_ckpt and n_ckpt > 0) else y.new_empty((0,), dtype=torch.float32)
        return torch.empty_like(y), ckpt

    @reg("sjb200::bn_lif_backward")
    def _(g_out, y, scale, shift, mean, invstd, gamma, ckpt, training, kind, tau, v_th, v_reset, soft_reset, v_init, sg_id, sg_p0,
          sg_p1, detach_reset):
        C = y.shape[-1]
        return torch.empty_like(y), y.new_empty((C,), dtype=torch.float32), y.new_empty((C,), dtype=torch.float32)

    @reg("sjb200::bn_pool_lif_forward")
    def _(y, scale, shift, T, is_static, kind, tau, v_th, v_reset, soft_reset, v_init):
        nb, h, w, c = y.shape
        oh, ow = (h - 1) // 2 + 1, (w - 1) // 2 + 1
        b = nb if is_static else nb // T
        return y.new_empty((T, b, oh, ow, c)), y.new_empty((nb, oh, ow, c), dtype=torch.uint8)

    @reg("sjb200::bn_pool_lif_backward")
    def _(g_out, y, idx, scale, shift, mean, invstd, gamma, training, T, is_static, kind, tau, v_th, v_reset, soft_reset, v_init,
          sg_id, sg_p0, sg_p1, detach_reset):
        C = y.shape[-1]
        return torch.empty_like(y), y.new_empty((C,), dtype=torch.float32), y.new_empty((C,), dtype=torch.float32)

    # ------------------------------------------------------------------ implicit-GEMM convolution
    def _conv_extent(size, pad, k, dil, stride):
        return (size + 2 * pad - dil * (k - 1) - 1) // stride + 1

    @reg("sjb200::conv2d_nhwc_forward")
    def _(x, w, stride, padding, dilation, want_stats):
        n, h, wd, _ = x.shape
        co, r, s_, _ = w.shape
        oh, ow = _conv_extent(h, padding[0], r, dilation[0], stride[0]), _conv_extent(wd, padding[1], s_, dilation[1], stride[1])
        rows = n * oh * ow
        stats = x.new_empty(((rows + 127) // 128 * 4, 2, co), dtype=torch.float32) if want_stats else x.new_empty((0,), dtype=torch.float32)
        return x.new_empty((rows, co)), stats

    @reg("sjb200::conv2d_nhwc_dgrad")
    def _(gy, w, H, W, stride, padding):
        co, r, s_, ci = w.shape
        oh, ow = _conv_extent(H, padding[0], r, 1, stride[0]), _conv_extent(W, padding[1], s_, 1, stride[1])
        return gy.new_empty((gy.numel() // (oh * ow * co), H, W, ci))

    @reg("sjb200::conv2d_nhwc_wgrad")
    def _(x, gy, R, S, stride, padding, dilation):
        n, h, wd, ci = x.shape
        oh, ow = _conv_extent(h, padding[0], R, dilation[0], stride[0]), _conv_extent(wd, padding[1], S, dilation[1], stride[1])
        return x.new_empty((gy.numel() // (n * oh * ow), R, S, ci), dtype=torch.float32)

    # ------------------------------------------------------------------ collectives and the fused tensor-parallel path
    @reg("sjb200::allreduce_bucket")
    def _(bucket, buf_ptrs, sig_ptrs, multicast_ptr, rank, epoch, scale, blocks, status, timeout_s, wire=0):
        return None

    @reg("sjb200::spike_gemm")
    def _(a_ptrs, a_pitch, M, K, w, rows_per_t, rows_per_src, rank, push_ptrs, slot_elems):
        # with push pointers the partial product is scattered to its owners and an empty tensor comes back
        return w.new_empty((0,)) if len(push_ptrs) > 0 else w.new_empty((M, w.shape[0]))

    @reg("sjb200::lif_pack")
    def _(x, out_ptr, pitch, tau, v_th):
        return None

    @reg("sjb200::rmsnorm_lif_pack")
    def _(h, weight, out_ptrs, pitch, eps, tau, v_th):
        return None

    @reg("sjb200::tp_reduce_residual")
    def _(h, stage_ptr, slot_elems, world):
        return None

    @reg("sjb200::tp_push_chunks")
    def _(src, dst_ptrs, chunks, dst_stride_bytes, dst_offset_bytes):
        return None

    @reg("sjb200::tp_reduce_chunks")
    def _(src_ptrs, out, chunks, src_stride_elems, src_offset_elems):
        return None

    @reg("sjb200::gemm_16bit_into")
    def _(a, b, a_mn, b_mn, out):
        return out

    @reg("sjb200::tp_barrier")
    def _(sig_ptrs, rank, epoch, status, timeout_s):
        return None
