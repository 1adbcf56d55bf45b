"""Implicit-GEMM convolution (``ops/conv.py``, ``csrc/conv_tcgen05.cu``) against ``F.conv2d`` in fp32 on the same
16-bit-rounded operands: forward, data gradient, weight gradient and the batch-norm partial sums."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

CASES = [
    # (N, C_in, H, W, C_out, k, stride, padding)
    (3, 64, 17, 13, 64, 3, 1, 1),          # odd extents, rows not a multiple of the 128-row tile
    (2, 64, 16, 16, 128, 3, 1, 1),
    (2, 128, 15, 15, 256, 3, 2, 1),        # stride 2, odd input
    (2, 128, 16, 16, 128, 3, 2, 1),        # stride 2, even input
    (1, 256, 9, 11, 512, 3, 1, 1),
    (1, 512, 7, 7, 512, 3, 1, 1),
    (2, 64, 16, 12, 128, 1, 2, 0),         # 1 x 1 stride 2 (ResNet downsample): three of four pixel classes get zero gradient
    (2, 64, 12, 20, 64, 3, 1, (2, 0)),     # asymmetric padding: tells the H and W corners of the gather apart
    (2, 64, 11, 11, 64, (3, 1), (1, 2), (1, 0)),
    (5, 64, 33, 31, 64, 3, 1, 1),          # several row tiles per image, images straddling tiles
]


def _pair(v):
    return tuple(v) if isinstance(v, (tuple, list)) else (v, v)


@pytest.mark.parametrize("case", CASES, ids=[str(c) for c in CASES])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_conv_forward_backward_match_fp32_reference(case, dtype):
    from spikingjelly_b200.ops import conv as C
    from spikingjelly_b200.ops import gemm as G
    N, ci, H, W, co, k, stride, padding = case
    if dtype == torch.float16 and case not in (CASES[0], CASES[2]):
        pytest.skip("fp16 is checked on two shapes")
    torch.manual_seed(0)
    dev = torch.device("cuda")
    kh, kw = _pair(k)
    x = (torch.rand(N, H, W, ci, device=dev) < 0.3).to(dtype)                     # spikes, NHWC
    w = (torch.randn(co, ci, kh, kw, device=dev) * 0.05).requires_grad_()
    xr = x.clone().requires_grad_()
    rows, stats, (oh, ow) = C.conv2d_rows(xr, w, stride, padding, 1, want_stats=True)
    G.check_status(rows)
    # reference in fp32 on the rounded operands
    x32 = x.float().permute(0, 3, 1, 2).contiguous().requires_grad_()
    w32 = w.detach().to(dtype).float().requires_grad_()
    ref = F.conv2d(x32, w32, None, _pair(stride), _pair(padding))
    assert ref.shape == (N, co, oh, ow)
    ref_rows = ref.permute(0, 2, 3, 1).reshape(-1, co)
    tol = 2e-2 if dtype == torch.bfloat16 else 4e-3
    torch.testing.assert_close(rows.float(), ref_rows, rtol=tol, atol=tol)
    # batch-norm partial sums are taken from the rounded result
    s1 = stats[:, 0].sum(0)
    s2 = stats[:, 1].sum(0)
    torch.testing.assert_close(s1, rows.float().sum(0), rtol=1e-3, atol=1e-2)
    torch.testing.assert_close(s2, (rows.float() ** 2).sum(0), rtol=1e-3, atol=1e-2)

    gy = torch.randn_like(rows)
    rows.backward(gy)
    G.check_status(rows)
    ref_rows.backward(gy.float())
    gx_ref = x32.grad.permute(0, 2, 3, 1)
    scale = gx_ref.abs().max().item()
    assert (xr.grad.float() - gx_ref).abs().max().item() <= tol * scale + 1e-3, "data gradient"
    gw_ref = w32.grad
    scale = gw_ref.abs().max().item()
    assert w.grad.shape == w.shape
    assert (w.grad - gw_ref).abs().max().item() <= 3e-3 * scale + 1e-3, "weight gradient"


def test_conv_is_deterministic_and_drop_in():
    from spikingjelly_b200.ops import conv as C
    torch.manual_seed(1)
    dev = torch.device("cuda")
    conv = torch.nn.Conv2d(64, 128, 3, 1, 1, bias=True).to(dev)
    x = (torch.rand(4, 64, 14, 14, device=dev) < 0.2).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    assert C.supports(conv, x)
    a = C.conv2d_channels_last(x, conv.weight, conv.bias, conv.stride, conv.padding)
    b = C.conv2d_channels_last(x, conv.weight, conv.bias, conv.stride, conv.padding)
    assert torch.equal(a, b) and a.shape == (4, 128, 14, 14) and a.is_contiguous(memory_format=torch.channels_last)
    ref = F.conv2d(x.float(), conv.weight.to(torch.bfloat16).float(), conv.bias, 1, 1)
    torch.testing.assert_close(a.float(), ref, rtol=2e-2, atol=2e-2)
    assert not C.supports(torch.nn.Conv2d(3, 64, 3).to(dev), x)                  # few input channels: the stem path's job
    assert not C.supports(torch.nn.Conv2d(64, 64, 3, groups=2).to(dev), x)


def test_spike_conv_and_linear_run_natively_and_keep_bits():
    """``cuda_kernel.spike_op``: 16-bit spike inputs go through the tensor-core kernels in all three passes and the
    input is kept as bits; results equal the library operators on the same rounded operands."""
    from spikingjelly_b200.activation_based.cuda_kernel import spike_op
    from spikingjelly_b200.ops import counters
    torch.manual_seed(2)
    dev = torch.device("cuda")
    conv = spike_op.SpikeConv2d(64, 128, 3, stride=2, padding=1, bias=True).to(dev)
    s = (torch.rand(3, 64, 13, 14, device=dev) < 0.25).to(torch.bfloat16).requires_grad_()
    counters.reset()
    y = conv(s)
    gy = torch.randn_like(y)
    y.backward(gy)
    assert counters.by_name().get("conv_tcgen05", 0) == 3 and counters.by_name().get("bit_pack", 0) == 1
    s32 = s.detach().float().requires_grad_()
    w32 = conv.weight.detach().to(torch.bfloat16).float().requires_grad_()
    b32 = conv.bias.detach().to(torch.bfloat16).float().requires_grad_()
    ref = F.conv2d(s32, w32, b32, 2, 1)
    ref.backward(gy.float())
    torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2)
    assert (s.grad.float() - s32.grad).abs().max() <= 2e-2 * s32.grad.abs().max() + 1e-3
    assert (conv.weight.grad - w32.grad).abs().max() <= 3e-3 * w32.grad.abs().max() + 1e-3
    assert (conv.bias.grad - b32.grad).abs().max() <= 2e-2 * b32.grad.abs().max() + 1e-2

    lin = spike_op.SpikeLinear(96, 40).to(dev)
    s = (torch.rand(4, 7, 96, device=dev) < 0.3).to(torch.float16).requires_grad_()
    with torch.autocast("cuda", dtype=torch.float16):
        y = lin(s)
    gy = torch.randn_like(y)
    y.backward(gy)
    s32 = s.detach().float().requires_grad_()
    w32 = lin.weight.detach().half().float().requires_grad_()
    ref = F.linear(s32, w32, lin.bias.detach().half().float())
    ref.backward(gy.float())
    torch.testing.assert_close(y.float(), ref, rtol=4e-3, atol=4e-3)
    torch.testing.assert_close(s.grad.float(), s32.grad, rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(lin.weight.grad, w32.grad, rtol=1e-2, atol=1e-2)
