"""Fused PSN operator against the eager formulation (addmm + surrogate): spikes identical, gradients of input, weight and
bias close; the three PSN modules take the fused path on CUDA."""
import pytest
import torch

from spikingjelly_b200.activation_based import functional, neuron, surrogate
from spikingjelly_b200.ops import counters, psn as psn_op

pytestmark = pytest.mark.gpu


def _eager(x, w, b, sg):
    return sg(torch.addmm(b.view(-1, 1), w, x.flatten(1))).view(x.shape)


@pytest.mark.parametrize("T", [1, 4, 7, 16, 32])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("with_sg", [False, True])
def test_matches_eager(T, dtype, with_sg):
    torch.manual_seed(T)
    sg = surrogate.ATan()
    x = (torch.randn(T, 6, 200, device="cuda") * 0.7).to(dtype).requires_grad_(True)
    w = (torch.randn(T, T, device="cuda") * 0.5).requires_grad_(True)
    b = (torch.randn(T, 1, device="cuda") * 0.1).requires_grad_(True)
    g = torch.randn(T, 6, 200, device="cuda").to(dtype)
    s = psn_op.psn_spikes(x, w, b, surrogate.surrogate_spec(sg), sg if with_sg else None)
    gx, gw, gb = torch.autograd.grad(s, (x, w, b), g)
    xr = x.detach().float().requires_grad_(True)
    wr, br = w.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    sr = _eager(xr, wr, br, sg)
    rx, rw, rb = torch.autograd.grad(sr, (xr, wr, br), g.float())
    h = torch.addmm(br.view(-1, 1), wr, xr.flatten(1)).view(x.shape).detach()
    sure = h.abs() > (1e-5 if dtype == torch.float32 else 1e-2)               # away from the threshold the spikes must agree
    assert torch.equal(s.float()[sure], sr.detach()[sure])
    cos = lambda a, c: torch.nn.functional.cosine_similarity(a.flatten().float(), c.flatten().float(), dim=0).item()
    tol = 0.9999 if dtype == torch.float32 else 0.995
    assert cos(gx, rx) > tol and cos(gw, rw) > tol and cos(gb, rb) > tol, (cos(gx, rx), cos(gw, rw), cos(gb, rb))
    assert gb.shape == b.shape and gw.dtype == w.dtype


def test_modules_take_the_fused_path():
    torch.manual_seed(0)
    x = torch.randn(8, 4, 64, device="cuda")
    for make in (lambda: neuron.PSN(8), lambda: neuron.MaskedPSN(3, 8, step_mode="m"), lambda: neuron.SlidingPSN(3, step_mode="m")):
        net = make().cuda()
        before = counters.by_name().get("psn_forward", 0)
        xin = x.clone().requires_grad_(True)
        out = net(xin)
        assert counters.by_name().get("psn_forward", 0) == before + 1
        out.sum().backward()
        assert xin.grad is not None and all(p.grad is not None for p in net.parameters() if p.requires_grad)
        ref = make().cuda()
        ref.load_state_dict(net.state_dict())
        xr = x.cpu().clone().requires_grad_(True)
        ref = ref.cpu()
        functional.reset_net(ref)
        outr = ref(xr)
        outr.sum().backward()
        assert (out.cpu() != outr).float().mean() < 1e-3
        for p, q in zip(net.parameters(), ref.parameters()):
            if p.grad is not None and q.grad is not None:
                assert torch.allclose(p.grad.cpu(), q.grad, rtol=1e-3, atol=1e-3)


def test_unsupported_inputs_fall_back():
    assert not psn_op.supported(torch.randn(40, 8, device="cuda"), (1, 2.0, 0.0))         # T > 32
    assert not psn_op.supported(torch.randn(4, 3, device="cuda"), (1, 2.0, 0.0))          # rows not 16-byte multiples
    assert not psn_op.supported(torch.randn(4, 8), (1, 2.0, 0.0))
    assert not psn_op.supported(torch.randn(4, 8, device="cuda"), None)
    net = neuron.PSN(4).cuda()
    assert net(torch.randn(4, 3, device="cuda")).shape == (4, 3)
