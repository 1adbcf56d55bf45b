"""Fused multi-step neuron kernels against the eager PyTorch fp32 rule on the same GPU.

Spikes and membrane potentials must be bit-identical in fp32 (the kernel uses
non-contracting arithmetic in the eager operation order); gradients agree to rounding."""
import itertools

import pytest
import torch

from spikingjelly_b200.activation_based import functional, neuron, surrogate

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _pair(cls, **kw):
    torch.manual_seed(0)
    a = cls(step_mode="m", backend="torch", **kw).to(DEV)
    b = cls(step_mode="m", backend="cuda", **kw).to(DEV)
    b.load_state_dict(a.state_dict())
    return a, b


def _run(net, x, gy, gv=None):
    x = x.clone().requires_grad_(True)
    y = net(x)
    loss = (y * gy).sum()
    if gv is not None:
        loss = loss + (net.v * gv).sum()
        if net.store_v_seq:
            loss = loss + (net.v_seq * 0.5).sum()
    loss.backward()
    return y.detach(), net.v.detach().clone(), x.grad.detach()


CASES = [
    (neuron.IFNode, {}),
    (neuron.LIFNode, {"tau": 2.0, "decay_input": True}),
    (neuron.LIFNode, {"tau": 3.7, "decay_input": False}),
    (neuron.ParametricLIFNode, {"init_tau": 2.0, "decay_input": True}),
    (neuron.ParametricLIFNode, {"init_tau": 4.0, "decay_input": False}),
    (neuron.QIFNode, {"tau": 2.0}),
    (neuron.EIFNode, {"tau": 2.0}),
]


@pytest.mark.parametrize("cls,kw", CASES)
@pytest.mark.parametrize("v_reset", [0.0, None])
@pytest.mark.parametrize("detach_reset", [False, True])
@pytest.mark.parametrize("T,N", [(1, 64), (4, 1000), (8, 4096), (16, 515), (20, 2048)])
def test_fp32_matches_eager(cls, kw, v_reset, detach_reset, T, N):
    if cls in (neuron.QIFNode, neuron.EIFNode) and v_reset is not None:
        v_reset = -0.1
    a, b = _pair(cls, v_reset=v_reset, detach_reset=detach_reset, surrogate_function=surrogate.ATan(), **kw)
    torch.manual_seed(1)
    x = torch.randn(T, 3, N, device=DEV) + 0.5
    if cls in (neuron.QIFNode, neuron.EIFNode):
        x = x * 0.3          # keeps the self-exciting dynamics finite under soft reset
    gy = torch.randn_like(x)
    gv = torch.randn(3, N, device=DEV)
    ya, va, ga = _run(a, x, gy, gv)
    yb, vb, gb = _run(b, x, gy, gv)
    exact = cls is not neuron.EIFNode   # expf differs from torch.exp in the last ulp
    if exact:
        assert torch.equal(ya, yb)
        assert torch.equal(va, vb)
    else:
        assert (ya != yb).float().mean() < 1e-3
    torch.testing.assert_close(gb, ga, rtol=2e-4 if exact else 5e-3, atol=2e-5 if exact else 1e-3)
    if cls is neuron.ParametricLIFNode:
        torch.testing.assert_close(b.w.grad, a.w.grad, rtol=2e-3, atol=1e-4)


@pytest.mark.parametrize("sg", [surrogate.Sigmoid(), surrogate.ATan(), surrogate.PiecewiseQuadratic(),
                                surrogate.PiecewiseExp(), surrogate.SoftSign(), surrogate.SuperSpike(),
                                surrogate.Erf(), surrogate.NonzeroSignLogAbs(), surrogate.PiecewiseLeakyReLU(),
                                surrogate.SquarewaveFourierSeries(n=3), surrogate.S2NN(), surrogate.QPseudoSpike(),
                                surrogate.LeakyKReLU(leak=0.1), surrogate.FakeNumericalGradient(),
                                surrogate.LogTailedReLU(alpha=0.1), surrogate.DeterministicPass(), surrogate.Rect()],
                         ids=lambda s: type(s).__name__)
def test_every_surrogate(sg):
    a, b = _pair(neuron.LIFNode, surrogate_function=sg)
    x = torch.randn(4, 2, 1024, device=DEV) + 0.5
    gy = torch.randn_like(x)
    ya, _, ga = _run(a, x, gy)
    yb, _, gb = _run(b, x, gy)
    assert torch.equal(ya, yb)
    torch.testing.assert_close(gb, ga, rtol=1e-3, atol=1e-4)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("N", [4096, 1001])
def test_half_precision(dtype, N):
    """Half storage, fp32 arithmetic inside the kernel: compare with the eager rule run in
    fp32 on the same (rounded) inputs."""
    b = neuron.LIFNode(step_mode="m", backend="cuda", surrogate_function=surrogate.ATan()).to(DEV)
    a = neuron.LIFNode(step_mode="m", backend="torch", surrogate_function=surrogate.ATan()).to(DEV)
    x = (torch.randn(8, 2, N, device=DEV) + 0.5).to(dtype)
    gy = torch.randn_like(x)
    ya, va, ga = _run(a, x.float(), gy.float())
    yb, vb, gb = _run(b, x, gy)
    assert yb.dtype == dtype and gb.dtype == dtype
    assert torch.equal(ya, yb.float())
    tol = 2e-2 if dtype is torch.bfloat16 else 3e-3
    torch.testing.assert_close(gb.float(), ga, rtol=tol, atol=tol)
    torch.testing.assert_close(vb.float(), va, rtol=tol, atol=tol)


def test_store_v_seq_and_state_carry():
    a, b = _pair(neuron.LIFNode, store_v_seq=True, surrogate_function=surrogate.Sigmoid())
    x = torch.randn(12, 4, 256, device=DEV) + 0.3
    for net in (a, b):
        net(x[:5])
        net(x[5:])       # state carried across calls
    assert torch.equal(a.v, b.v)
    assert torch.equal(a.v_seq, b.v_seq)
    functional.reset_net(b)
    assert b.v == 0.0 and b.v_seq is None


def test_single_step_native():
    a = neuron.LIFNode(backend="torch").to(DEV)
    b = neuron.LIFNode(backend="cuda").to(DEV)
    x = torch.randn(5, 3, 77, device=DEV) + 0.5
    for t in range(5):
        assert torch.equal(a(x[t]), b(x[t]))
    assert torch.equal(a.v, b.v)


def test_bit_packed_spikes():
    from spikingjelly_b200.ops.neuron_scan import KIND, NeuronSpec, multistep_neuron
    for N, dt in [(4096, torch.float32), (4096, torch.bfloat16), (1000, torch.float32), (72, torch.float16)]:
        x = (torch.randn(4, N, device=DEV) + 0.5).to(dt)
        spec = NeuronSpec(KIND["lif_di"], 1.0, 0.0, 2.0)
        s, _, _, packed = multistep_neuron(x, 0.0, spec, pack_bits=True)
        words = packed.view(torch.int32).cpu().numpy().astype("uint32")
        import numpy as np
        bits = np.unpackbits(words.view(np.uint8).reshape(4, -1), axis=1, bitorder="little")[:, :N]
        assert (bits == s.float().cpu().numpy().astype(np.uint8)).all()


def test_deterministic_twice():
    b = neuron.ParametricLIFNode(step_mode="m", backend="cuda").to(DEV)
    x = torch.randn(8, 1 << 16, device=DEV)
    gy = torch.randn_like(x)
    outs = []
    for _ in range(2):
        b.w.grad = None
        functional.reset_net(b)
        _, _, g = _run(b, x, gy)
        outs.append((g, b.w.grad.clone()))
    assert torch.equal(outs[0][0], outs[1][0])
    assert torch.equal(outs[0][1], outs[1][1])


@pytest.mark.gpu
@pytest.mark.parametrize("T,N", [(4, 4096), (8, 4096), (16, 1000), (5, 777)])
@pytest.mark.parametrize("kind", ["if", "lif_di", "lif_ndi"])
@pytest.mark.parametrize("storage", [torch.float8_e4m3fn, torch.float8_e5m2])
def test_fp8_input_equals_bf16_kernel_on_the_same_values(T, N, kind, storage):
    """x stored as one byte per element (e4m3 or e5m2): every fp8 value is exact in bf16, so spikes, final potential and
    the input gradient must be bit-identical to the bf16 kernel fed with the widened tensor."""
    from spikingjelly_b200 import ops
    from spikingjelly_b200.ops.neuron_scan import KIND
    ops.require()
    torch.manual_seed(0)
    x8 = (torch.randn(T, N, device="cuda") + 0.5).to(storage)
    x16 = x8.to(torch.bfloat16)
    g = torch.randn(T, N, device="cuda").to(torch.bfloat16)
    k = KIND[kind]

    def run(x):
        s, v, _, _, ck = torch.ops.sjb200.scan_forward(x, None, 0.0, None, k, 2.0, 0.0, 0.0, 0.0, 1.0, 0.0, False, False, False, True)
        gx, _, _ = torch.ops.sjb200.scan_backward(g, None, None, x, None, 0.0, None, ck if ck.numel() else None, k, 2.0, 0.0, 0.0, 0.0,
                                                  1.0, 0.0, False, 1, 2.0, 0.0, False, False)
        return s, v, gx

    a, b = run(x8), run(x16)
    assert a[0].dtype == torch.bfloat16 and a[2].dtype == torch.bfloat16
    for u, w in zip(a, b):
        assert torch.equal(u, w)
