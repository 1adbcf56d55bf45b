"""Fused BatchNorm + LIF against torch BatchNorm followed by the eager LIF rule (fp32)."""
import pytest
import torch
import torch.nn as nn

from spikingjelly_b200.activation_based import functional, neuron, surrogate
from spikingjelly_b200.ops.bn_lif import bn_lif
from spikingjelly_b200.ops.neuron_scan import KIND, NeuronSpec

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _reference(y, bn, lif, residual):
    """y: [T, R, C] -> torch BN over (T*R) per channel, then LIF over T."""
    T, R, C = y.shape
    z = bn(y.reshape(T * R, C)).reshape(T, R, C)
    out = lif(z)
    return out + residual if residual is not None else out


@pytest.mark.parametrize("T,R,C", [(4, 196, 64), (4, 1000, 512), (6, 77, 1536), (1, 33, 8)])
@pytest.mark.parametrize("with_res", [False, True])
@pytest.mark.parametrize("training", [True, False])
def test_matches_unfused_fp32(T, R, C, with_res, training):
    torch.manual_seed(0)
    bn_a, bn_b = nn.BatchNorm1d(C).to(DEV), nn.BatchNorm1d(C).to(DEV)
    with torch.no_grad():
        bn_a.weight.uniform_(0.5, 1.5); bn_a.bias.uniform_(-0.2, 0.6)
        bn_a.running_mean.uniform_(-0.1, 0.1); bn_a.running_var.uniform_(0.5, 1.5)
    bn_b.load_state_dict(bn_a.state_dict())
    bn_a.train(training); bn_b.train(training)
    lif = neuron.LIFNode(tau=2.0, detach_reset=True, step_mode="m", surrogate_function=surrogate.Sigmoid()).to(DEV)
    spec = NeuronSpec(KIND["lif_di"], 1.0, 0.0, 2.0, sg=surrogate.Sigmoid().kernel_spec(), detach_reset=True)
    y = (torch.randn(T, R, C, device=DEV) * 1.3 + 0.2)
    res = torch.randint(0, 3, (T, R, C), device=DEV).float() if with_res else None
    g = torch.randn(T, R, C, device=DEV)

    ya = y.clone().requires_grad_(True)
    oa = _reference(ya, bn_a, lif, res)
    oa.backward(g)
    functional.reset_net(lif)
    yb = y.clone().requires_grad_(True)
    ob = bn_lif(yb, bn_b, spec, residual=res)
    ob.backward(g)

    flips = (oa != ob).float().mean().item()
    assert flips < 2e-4, f"fraction of differing spikes {flips}"
    if flips == 0:
        torch.testing.assert_close(yb.grad, ya.grad, rtol=2e-3, atol=2e-4)
        torch.testing.assert_close(bn_b.weight.grad, bn_a.weight.grad, rtol=2e-3, atol=2e-3)
        torch.testing.assert_close(bn_b.bias.grad, bn_a.bias.grad, rtol=2e-3, atol=2e-3)
    torch.testing.assert_close(bn_b.running_mean, bn_a.running_mean, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(bn_b.running_var, bn_a.running_var, rtol=1e-4, atol=1e-5)
    assert int(bn_b.num_batches_tracked) == int(bn_a.num_batches_tracked)


def test_bf16_close_to_fp32_path():
    torch.manual_seed(1)
    T, R, C = 4, 512, 256
    bn = nn.BatchNorm1d(C).to(DEV)
    spec = NeuronSpec(KIND["lif_di"], 1.0, 0.0, 2.0, sg=surrogate.Sigmoid().kernel_spec(), detach_reset=True)
    y = torch.randn(T, R, C, device=DEV).to(torch.bfloat16)
    g = torch.randn(T, R, C, device=DEV).to(torch.bfloat16)
    y16 = y.clone().requires_grad_(True)
    o16 = bn_lif(y16, bn, spec)
    o16.backward(g)
    bn2 = nn.BatchNorm1d(C).to(DEV)
    y32 = y.float().requires_grad_(True)
    o32 = bn_lif(y32, bn2, spec)
    o32.backward(g.float())
    assert o16.dtype == torch.bfloat16
    assert (o16.float() != o32).float().mean() < 1e-4
    torch.testing.assert_close(y16.grad.float(), y32.grad, rtol=5e-2, atol=2e-2)


def test_deterministic():
    T, R, C = 4, 3000, 128
    bn = nn.BatchNorm1d(C).to(DEV)
    spec = NeuronSpec(KIND["lif_di"], 1.0, 0.0, 2.0, sg=surrogate.ATan().kernel_spec())
    y = torch.randn(T, R, C, device=DEV)
    g = torch.randn(T, R, C, device=DEV)
    grads = []
    for _ in range(2):
        yy = y.clone().requires_grad_(True)
        bn.weight.grad = None
        bn_lif(yy, bn, spec).backward(g)
        grads.append((yy.grad.clone(), bn.weight.grad.clone()))
    assert torch.equal(grads[0][0], grads[1][0]) and torch.equal(grads[0][1], grads[1][1])
