"""Lava / Lynxi / NIR exchange layers without the vendor packages: arithmetic, rewrites and parameter round trips."""
import numpy as np
import pytest
import torch
import torch.nn as nn

from spikingjelly_b200.activation_based import functional, layer, lava_exchange as L, lynxi_exchange as X, neuron
from spikingjelly_b200.activation_based.nir_exchange import module_to_spec, spec_to_module


def test_lava_quantisers_and_integer_leak():
    w = torch.tensor([0.013, -0.5, 3.99, -4.2, 5.0])
    q = L.quantize_8b(w, 64)
    assert torch.allclose(q[:2] * 32, torch.round(q[:2] * 32)) and q.max() == 255 / 64 and q.min() == -4.0
    assert torch.equal(L.quantize_8b(w, 64, descale=True), q * 64)
    assert L.right_shift_to_zero(torch.tensor([-5, 5, -4, 7]), 1).tolist() == [-2, 2, -2, 3]
    x = torch.tensor([0.5, -0.25], requires_grad=True)
    state = torch.tensor([1.0, -1.0], requires_grad=True)
    decay = torch.tensor(1024.0, requires_grad=True)                    # a quarter
    y = L.LeakyIntegratorStep.apply(x, decay, state, 4096)
    assert torch.allclose(y, torch.tensor([1.25, -1.0]))
    y.sum().backward()
    assert torch.allclose(state.grad, torch.full((2,), 0.75)) and torch.allclose(x.grad, torch.ones(2))
    assert torch.allclose(decay.grad, -(state.detach() / 4096).sum())


def test_cuba_lif_node_dynamics_and_block_container():
    n = L.CubaLIFNode(current_decay=1.0, voltage_decay=0.0, step_mode="m", store_v_seq=True, store_i_seq=True)     # an IF neuron
    x = torch.full((6, 2), 0.4)
    s = n(x)
    assert s[:, 0].tolist() == [0, 0, 1, 0, 0, 1] and n.i_seq.shape == (6, 2) and torch.allclose(n.i_seq, x, atol=1 / 4096)
    functional.reset_net(n)
    assert n.i_seq is None and n.current_state == 0.0
    blk = L.BlockContainer(nn.Linear(4, 3, bias=False), neuron.LIFNode(tau=2.0, decay_input=False), step_mode="m")
    assert isinstance(blk.neuron, L.CubaLIFNode) and blk.neuron.voltage_decay.item() == 2048.0
    out = blk(torch.rand(5, 2, 4))
    assert out.shape == (5, 2, 3)
    out.sum().backward()
    assert blk.synapse.weight.grad is not None
    with pytest.raises(ValueError):
        L.to_lava_neuron_param_dict(neuron.LIFNode(decay_input=True))
    assert L.to_lava_neuron_param_dict(neuron.IFNode())["voltage_decay"] == 0.0
    pool = L.SumPool2d(2)
    assert torch.allclose(pool(torch.ones(1, 1, 4, 4)), torch.full((1, 1, 2, 2), 4.0))
    assert torch.allclose(L.SumPool2d(2, dilation=2)(torch.ones(1, 2, 5, 5)), torch.full((1, 2, 1, 1), 4.0))
    if L.slayer is None:
        with pytest.raises(ImportError):
            blk.to_lava_block()
    assert L.NXT_to_TNX(L.TNX_to_NXT(torch.rand(3, 2, 4, 5))).shape == (3, 2, 4, 5)


def test_lynxi_rewrite_matches_stateful_modules():
    torch.manual_seed(0)
    T = 4
    net = nn.Sequential(layer.Conv2d(2, 4, 3, padding=1), layer.BatchNorm2d(4), neuron.LIFNode(tau=3.0), layer.MaxPool2d(2),
                        layer.Flatten(), layer.Linear(4 * 4 * 4, 5), neuron.IFNode())
    functional.set_step_mode(net, "m")
    net.eval()
    out = X.to_lynxi_supported_modules(net, T)
    assert isinstance(out[0], nn.Conv2d) and isinstance(out[2], X.LIFNode) and isinstance(out[6], X.IFNode) and isinstance(out[3], nn.MaxPool2d)
    lynxi = nn.Sequential(*out).eval()
    x = torch.rand(T, 3, 2, 8, 8)
    with torch.no_grad():
        ref = net(x)
        got = lynxi(x.flatten(0, 1)).view(T, 3, 5)                       # time folded into the batch
    assert torch.equal(ref, got)
    s, v = X.LIFNode(tau=2.0, v_reset=None, return_v=True)(torch.tensor([3.0]))
    assert s.item() == 1.0 and v.item() == 0.5
    with pytest.raises(ImportError):
        X.load_lynxi_model(0, "nowhere")


def test_nir_parameter_round_trip():
    dt = 1e-4
    lif = neuron.LIFNode(tau=5.0, decay_input=False, v_threshold=0.7, v_reset=0.0, step_mode="m")
    kind, p = module_to_spec(lif, (4, 2, 8, 3), (4, 2, 8, 3), dt)
    assert kind == "LIF" and p["tau"].shape == (8, 3) and np.allclose(p["tau"], 5e-4) and np.allclose(p["r"], 5.0)
    back = spec_to_module(kind, p, dt)
    assert isinstance(back, neuron.LIFNode) and abs(back.tau - 5.0) < 1e-9 and back.decay_input is False and back.v_threshold == 0.7
    kind, p = module_to_spec(neuron.LIFNode(tau=2.0, decay_input=True), (2, 6), (2, 6), dt)
    assert np.allclose(p["r"], 1.0) and spec_to_module(kind, p, dt).decay_input is True
    kind, p = module_to_spec(neuron.IFNode(v_reset=None), (2, 6), (2, 6), dt)
    assert kind == "IF" and np.allclose(p["r"], 1e4) and np.allclose(p["v_reset"], 0.0)
    assert isinstance(spec_to_module(kind, p, dt), neuron.IFNode)
    with pytest.raises(AssertionError):
        spec_to_module("IF", {**p, "r": np.full((6,), 3.0)}, dt)
    conv = layer.Conv2d(4, 6, 3, stride=2, padding=1, groups=2, bias=False)
    kind, p = module_to_spec(conv, (2, 4, 9, 9), (2, 6, 5, 5), dt)
    c2 = spec_to_module(kind, p, dt)
    assert p["input_shape"] == (9, 9) and c2.in_channels == 4 and c2.groups == 2 and torch.equal(c2.weight, conv.weight) and torch.all(c2.bias == 0)
    kind, p = module_to_spec(layer.Flatten(1, step_mode="m") if "step_mode" in layer.Flatten.__init__.__code__.co_varnames else layer.Flatten(1), (3, 2, 4, 5), (3, 2, 20), dt)
    assert kind == "Flatten" and p["start_dim"] == 0 and spec_to_module(kind, p, dt).start_dim == 1
    kind, p = module_to_spec(nn.Linear(3, 2), (1, 3), (1, 2), dt)
    assert kind == "Affine" and spec_to_module(kind, p, dt).weight.shape == (2, 3)
    from spikingjelly_b200.activation_based import nir_exchange
    with pytest.raises(ImportError):
        nir_exchange.export_to_nir(nn.Sequential(nn.Linear(3, 2)), torch.zeros(1, 3))
