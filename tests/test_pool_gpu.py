"""Channels-last 3 x 3 / 2 max pooling against ``torch.nn.functional.max_pool2d`` in fp32 (values, tie rule, gradient)."""
import pytest
import torch
import torch.nn.functional as F

from spikingjelly_b200 import ops
from spikingjelly_b200.ops import pool

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True)
def _lib():
    ops.require()


@pytest.mark.parametrize("N,C,H,W", [(3, 64, 16, 16), (2, 8, 15, 9), (4, 128, 7, 12), (1, 16, 1, 1)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("spikes", [True, False])
def test_matches_library_pool(N, C, H, W, dtype, spikes):
    torch.manual_seed(0)
    x = (torch.rand(N, C, H, W, device=DEV) < 0.3).to(dtype) if spikes else torch.randn(N, C, H, W, device=DEV).to(dtype)
    x = x.contiguous(memory_format=torch.channels_last).requires_grad_(True)
    mp = torch.nn.MaxPool2d(3, 2, 1)
    assert pool.supports(mp, x)
    y = pool.max_pool_3x3s2_channels_last(x)
    xr = x.detach().float().requires_grad_(True)
    yr = F.max_pool2d(xr, 3, 2, 1)
    assert y.shape == yr.shape and y.is_contiguous(memory_format=torch.channels_last)
    torch.testing.assert_close(y.float(), yr, rtol=0, atol=0)
    g = torch.randn_like(yr)
    y.backward(g.to(dtype))
    yr.backward(g.to(dtype).float())
    # ties (spike maps are full of them) must resolve to the same window element as the library kernel
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=1e-2, atol=1e-2)


def test_not_supported_cases_fall_through():
    x = torch.randn(2, 8, 8, 8, device=DEV).to(torch.bfloat16)
    assert not pool.supports(torch.nn.MaxPool2d(3, 2, 1), x)                       # NCHW strides
    xc = x.contiguous(memory_format=torch.channels_last)
    assert not pool.supports(torch.nn.MaxPool2d(2, 2), xc)
    assert not pool.supports(torch.nn.MaxPool2d(3, 2, 1, ceil_mode=True), xc)
    assert not pool.supports(torch.nn.MaxPool2d(3, 2, 1), xc.float())


@pytest.mark.parametrize("N,Ci,H,W,Co,k,s,p", [(4, 2, 32, 32, 64, 7, 2, 3), (2, 3, 17, 23, 16, 3, 1, 1), (3, 1, 9, 9, 8, 5, 2, 0)])
def test_few_channel_convolution_matches_conv2d(N, Ci, H, W, Co, k, s, p):
    from spikingjelly_b200.ops import conv_stem
    torch.manual_seed(0)
    x = torch.randn(N, Ci, H, W, device=DEV).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    conv = torch.nn.Conv2d(Ci, Co, k, s, p, bias=False).to(DEV)
    assert conv_stem.supports(conv, x)
    rows, stats, (oh, ow) = conv_stem.conv2d_few_channels(x, conv.weight, conv.stride, conv.padding)
    y = rows.view(N, oh, ow, Co).permute(0, 3, 1, 2)
    wr = conv.weight.detach().to(torch.bfloat16).float().requires_grad_(True)
    yr = F.conv2d(x.float(), wr, None, s, p)
    torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=2e-2)
    yd = rows.detach().double()
    torch.testing.assert_close(stats[:, 0].double().sum(0), yd.sum(0), rtol=1e-5, atol=1e-3)
    g = torch.randn_like(yr)
    rows.backward(g.permute(0, 2, 3, 1).reshape(-1, Co).to(torch.bfloat16))
    yr.backward(g.to(torch.bfloat16).float())
    torch.testing.assert_close(conv.weight.grad, wr.grad, rtol=3e-2, atol=3e-2 * float(wr.grad.abs().max()))
