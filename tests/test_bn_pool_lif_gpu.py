"""Fused BN -> MaxPool(3,2,1) -> LIF stem kernel against the unfused PyTorch pipeline in fp32."""
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from spikingjelly_b200.activation_based import functional, neuron, surrogate
from spikingjelly_b200.ops.bn_lif import bn_pool_lif
from spikingjelly_b200.ops.neuron_scan import KIND, NeuronSpec

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("static", [True, False])
@pytest.mark.parametrize("T,B,H,W,C", [(4, 3, 16, 16, 64), (2, 2, 15, 9, 8), (6, 2, 8, 8, 128)])
def test_matches_unfused(static, T, B, H, W, C):
    torch.manual_seed(0)
    NB = B if static else T * B
    y16 = (torch.randn(NB, H, W, C, device=DEV) * 1.5 + 0.3).to(torch.bfloat16)
    bn_a, bn_b = nn.BatchNorm2d(C).to(DEV), nn.BatchNorm2d(C).to(DEV)
    with torch.no_grad():
        bn_a.weight.uniform_(0.5, 1.5); bn_a.bias.uniform_(-0.2, 0.5)
    bn_b.load_state_dict(bn_a.state_dict())
    lif = neuron.LIFNode(tau=2.0, detach_reset=True, step_mode="m", surrogate_function=surrogate.Sigmoid()).to(DEV)
    spec = NeuronSpec(KIND["lif_di"], 1.0, 0.0, 2.0, sg=surrogate.Sigmoid().kernel_spec(), detach_reset=True)
    OH, OW = (H - 1) // 2 + 1, (W - 1) // 2 + 1
    g = torch.randn(T, B, OH, OW, C, device=DEV)

    ya = y16.float().requires_grad_(True)
    z = bn_a(ya.permute(0, 3, 1, 2))
    p = F.max_pool2d(z, 3, 2, 1).permute(0, 2, 3, 1)
    seq = p.unsqueeze(0).expand(T, -1, -1, -1, -1) if static else p.reshape(T, B, OH, OW, C)
    oa = lif(seq)
    (oa * g).sum().backward()
    functional.reset_net(lif)

    yb = y16.clone().requires_grad_(True)
    ob = bn_pool_lif(yb, bn_b, spec, T, static)
    (ob.float() * g).sum().backward()

    assert ob.shape == (T, B, OH, OW, C)
    flips = (oa != ob.float()).float().mean().item()
    assert flips < 1e-3, flips
    if flips == 0:
        torch.testing.assert_close(yb.grad.float(), ya.grad, rtol=3e-2, atol=3e-2)
        torch.testing.assert_close(bn_b.weight.grad, bn_a.weight.grad, rtol=3e-2, atol=0.2)   # pooled gradient is stored in bf16
        torch.testing.assert_close(bn_b.bias.grad, bn_a.bias.grad, rtol=3e-2, atol=0.2)
    torch.testing.assert_close(bn_b.running_mean, bn_a.running_mean, rtol=1e-3, atol=1e-4)


def test_gradient_sum_is_conserved():
    """Every pooled gradient lands on exactly one input pixel: with frozen BN (pure affine), the
    per-channel sum of dy equals scale * sum of the pooled gradients."""
    T, B, H, W, C = 4, 2, 12, 12, 16
    y = torch.randn(T * B, H, W, C, device=DEV).to(torch.bfloat16).requires_grad_(True)
    bn = nn.BatchNorm2d(C).to(DEV).eval()
    with torch.no_grad():
        bn.running_var.fill_(1.0); bn.weight.fill_(1.0)
    spec = NeuronSpec(KIND["if"], 1.0, None, sg=surrogate.DeterministicPass().kernel_spec(), detach_reset=True)
    out = bn_pool_lif(y, bn, spec, T, False)
    out.float().sum().backward()
    # IF with pass-through surrogate and detached soft reset: dL/dx_t = T - t contributions of ones
    expected = sum(T - t for t in range(T)) * B * out.shape[2] * out.shape[3]
    per_channel = y.grad.float().sum(dim=(0, 1, 2))
    torch.testing.assert_close(per_channel, torch.full_like(per_channel, float(expected)) / (1 + 1e-5) ** 0.5,
                               rtol=2e-2, atol=1.0)
