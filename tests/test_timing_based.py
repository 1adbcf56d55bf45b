"""Tempotron and Gaussian tuning against closed-form expectations."""
import math

import pytest
import torch

from spikingjelly_b200.timing_based import encoding, neuron, orig_neuron


def test_tempotron_kernel_peaks_at_threshold_and_shapes():
    m = neuron.Tempotron(1, 1, T=100, tau=15.0, tau_s=15.0 / 4, v_threshold=1.0)
    with torch.no_grad():
        m.model.summation_layer.weight.fill_(1.0)
    v = m(torch.tensor([[0.0]]), "v")
    t_peak = 15.0 * (15.0 / 4) * math.log(4.0) / (15.0 - 15.0 / 4)
    assert v.shape == (1, 1, 100) and abs(v.argmax().item() - t_peak) <= 1 and v.max() <= 1.0 + 1e-6 and v.max() > 0.99
    assert torch.all(m(torch.tensor([[-1.0]]), "v") == 0)                 # a negative time is "no spike"
    assert list(m.state_dict()) == ["model.summation_layer.weight"]
    with pytest.raises(ValueError):
        m(torch.tensor([[0.0]]), "bad")
    with pytest.raises(ValueError):
        neuron.Tempotron(2, 2, 10, tau=3.0, tau_s=3.0)


def test_tempotron_spike_times_gradient_and_loss():
    torch.manual_seed(0)
    m = neuron.Tempotron(8, 3, T=30)
    x = torch.randint(-1, 30, (4, 8)).float()
    s = m(x, "spikes")
    v = m(x, "v")
    fired = v.max(2).values >= m.v_threshold
    assert torch.equal(s.abs().round(), v.argmax(2).float()) and torch.equal(s >= 0, fired | (v.argmax(2) == 0) & ~fired | fired)
    s.sum().backward()
    assert m.model.summation_layer.weight.grad.abs().sum() > 0
    label = torch.tensor([0, 1, 2, 0])
    vmax = m(x, "v_max")
    wrong = (fired.float() != torch.nn.functional.one_hot(label, 3)).float()
    assert torch.allclose(m.mse_loss(vmax, label), (((vmax - 1.0) * wrong) ** 2).sum() / 4)
    legacy = orig_neuron.Tempotron(8, 3, T=30)
    legacy.fc.load_state_dict(m.model.summation_layer.state_dict())
    assert list(legacy.state_dict()) == ["fc.weight"] and torch.allclose(legacy(x, "v"), v)
    assert torch.allclose(orig_neuron.Tempotron.mse_loss(vmax, 1.0, label, 3), m.mse_loss(vmax, label))


def test_gaussian_tuning():
    g = encoding.GaussianTuning(n=2, m=6, x_min=torch.zeros(2), x_max=torch.tensor([1.0, 4.0]))
    assert g.mu.shape == (2, 6) and torch.allclose(g.mu[0, 1], torch.tensor(1 / 8)) and torch.allclose(g.mu[1, -1] - g.mu[1, 0], torch.tensor(5.0))
    x = torch.stack([g.mu[0, 2].repeat(3), g.mu[1, 4].repeat(3)])[None]       # values sitting on a centre fire at t = 0
    t = g.encode(x, max_spike_time=50)
    assert t.shape == (1, 2, 3, 6) and torch.all(t[0, 0, :, 2] == 0) and torch.all(t[0, 1, :, 4] == 0)
    assert torch.all((t == -1) | ((t >= 0) & (t < 50))) and (t == -1).any()
    with pytest.raises(ValueError):
        encoding.GaussianTuning(2, 2, torch.zeros(2), torch.ones(2))
    with pytest.raises(AssertionError):
        g.encode(torch.zeros(1, 3, 4))
