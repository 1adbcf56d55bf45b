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
    def _(a, b, alpha, out_f32, split_k):
        return a.new_empty((a.shape[0], b.shape[0]), dtype=torch.float32 if out_f32 else torch.bfloat16)

    @reg("sjb200::fp8_quantize")
    def _(x, e5m2):
        return x.new_empty(x.shape, dtype=torch.float8_e5m2 if e5m2 else torch.float8_e4m3fn), x.new_empty((1,), dtype=torch.float32)

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
