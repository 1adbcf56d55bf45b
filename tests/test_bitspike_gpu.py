"""Bit-only spike output of the neuron scan: the bits equal the dense kernel's spikes, gradients through ``dense()`` and
``bit_linear`` equal the dense path's."""
import pytest
import torch

from spikingjelly_b200.ops import bitspike, neuron_scan
from spikingjelly_b200.ops.neuron_scan import KIND, NeuronSpec

pytestmark = pytest.mark.gpu


def _spec(kind="lif_di", soft=False):
    return NeuronSpec(kind=KIND[kind], v_threshold=1.0, v_reset=None if soft else 0.0, tau=2.0, sg=(1, 2.0, 0.0))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,shape", [(4, (8, 256)), (8, (3, 96)), (5, (7, 33))])
@pytest.mark.parametrize("kind,soft", [("lif_di", False), ("if", True)])
def test_bits_equal_dense_spikes_and_gradients(dtype, T, shape, kind, soft):
    torch.manual_seed(0)
    spec = _spec(kind, soft)
    x = (torch.randn(T, *shape, device="cuda") + 0.3).to(dtype)
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    dense, v_a, _, _ = neuron_scan.multistep_neuron(xa, 0.0, spec)
    bits, v_b = bitspike.multistep_neuron_bits(xb, 0.0, spec)
    assert bits.words.dtype == torch.int32 and bits.words.shape == (T, (x[0].numel() + 31) // 32)
    assert bits.handle.shape == x.shape and bits.handle.untyped_storage().nbytes() <= 8
    got = bits.dense()
    assert got.dtype == dense.dtype and torch.equal(got, dense) and torch.equal(v_a, v_b)
    g = torch.randn_like(dense)
    dense.backward(g)
    got.backward(g)
    assert torch.equal(xa.grad, xb.grad)


def test_bit_linear_matches_dense_linear():
    torch.manual_seed(1)
    spec = _spec()
    x = (torch.randn(4, 16, 256, device="cuda") + 0.3).to(torch.bfloat16)
    w = (torch.randn(128, 256, device="cuda") * 0.05).requires_grad_(True)
    b = torch.zeros(128, device="cuda", requires_grad=True)
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    dense, _, _, _ = neuron_scan.multistep_neuron(xa, 0.0, spec)
    ya = torch.nn.functional.linear(dense.float(), w, b)
    bits, _ = bitspike.multistep_neuron_bits(xb, 0.0, spec)
    yb = bitspike.bit_linear(bits, w, b)
    assert yb.shape == ya.shape and torch.allclose(yb.float(), ya, rtol=2e-2, atol=2e-2)
    g = torch.randn_like(ya)
    ga = torch.autograd.grad(ya, (xa, w, b), g)
    gb = torch.autograd.grad(yb, (xb, w, b), g.to(yb.dtype))
    cos = lambda u, v: torch.nn.functional.cosine_similarity(u.flatten().float(), v.flatten().float(), dim=0).item()
    assert cos(ga[0], gb[0]) > 0.995 and cos(ga[1], gb[1]) > 0.999 and cos(ga[2], gb[2]) > 0.999
