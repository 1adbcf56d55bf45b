"""``layer.misc`` and the OTTT layers: own expectations on CPU, and equality with the reference package where it is installed."""
import pytest
import torch
import torch.nn as nn

from spikingjelly_b200.activation_based import functional, layer


def test_synapse_filter_delay_and_voting():
    torch.manual_seed(0)
    s = (torch.rand(6, 3, 5) < 0.4).float()
    f = layer.SynapseFilter(tau=4.0, step_mode="m")
    out = f(s)
    i = torch.zeros(3, 5)
    for t in range(6):
        i = i - (1.0 - s[t]) * i / 4.0 + s[t]
        torch.testing.assert_close(out[t], i)
    functional.reset_net(f)
    learn = layer.SynapseFilter(tau=4.0, learnable=True, step_mode="m")
    torch.testing.assert_close(learn(s), out)                       # 1 / tau = sigmoid(w) with w = -log(tau - 1)
    learn(s[:2]).sum().backward()
    assert learn.w.grad is not None and "tau=4" in learn.extra_repr()[:8]

    d = layer.Delay(2, step_mode="m")
    x = torch.arange(5.0).view(5, 1)
    assert d(x).flatten().tolist() == [0.0, 0.0, 0.0, 1.0, 2.0]
    d.step_mode = "s"
    assert float(d(torch.tensor([9.0]))) == 3.0 and float(d(torch.tensor([9.0]))) == 4.0   # the queue carried over

    v = layer.VotingLayer(voting_size=2, step_mode="m")
    y = v(torch.tensor([[[1.0, 3.0, 0.0, 2.0]]]))
    assert y.tolist() == [[[2.0, 1.0]]]


def test_count_to_binary_round_trip_and_gradient():
    counts = torch.tensor([[[0.0, 3.0], [2.0, 1.0]]], requires_grad=True)            # [T=1, N=2, 2]
    expand, fold = layer.SpikeCountToBinary(3, always_convert=True), layer.TemporalBinSum(3, always_convert=True)
    b = expand(counts)
    assert b.shape == (3, 2, 2) and set(b.detach().unique().tolist()) <= {0.0, 1.0}
    assert b[:, 0, 1].tolist() == [1.0, 1.0, 1.0] and b[:, 1, 0].tolist() == [1.0, 1.0, 0.0]
    torch.testing.assert_close(fold(b), counts.detach())
    b.sum().backward()
    torch.testing.assert_close(counts.grad, torch.ones_like(counts))                 # 3 sub-steps x (1 / 3)
    assert layer.TemporalBinSum(4, always_convert=True)(torch.ones(6, 1, 1)).flatten().tolist() == [4.0, 2.0]
    assert expand.train()(counts) is not None and layer.SpikeCountToBinary(3).train()(counts) is counts
    with pytest.raises(ValueError):
        layer.SpikeCountToBinary(0)
    with pytest.raises(ValueError):
        fold(torch.ones(3))


def test_ottt_sequential_routes_gradients_through_the_trace():
    torch.manual_seed(1)
    lin = nn.Linear(4, 3)
    net = layer.OTTTSequential(nn.Flatten(), lin)
    spike = (torch.rand(2, 2, 2) < 0.5).float()
    trace = torch.rand(2, 2, 2)
    out = net([spike, trace])
    torch.testing.assert_close(out, lin(spike.flatten(1)))                           # value from the spike
    g = torch.rand_like(out)
    out.backward(g)
    torch.testing.assert_close(lin.weight.grad, g.t() @ trace.flatten(1))            # weight gradient from the trace
    pair = layer.SpikeTraceOp(nn.Flatten())([spike, trace])
    assert isinstance(pair, list) and pair[0].shape == (2, 4) and not pair[1].requires_grad
    assert layer.GradwithTrace(lin)([spike.flatten(1), trace.flatten(1)]).shape == (2, 3)


def test_equal_to_reference_layers(reference):
    torch.manual_seed(2)
    s = (torch.rand(5, 2, 6) < 0.5).float()
    for ours, theirs in ((layer.SynapseFilter(3.0, step_mode="m"), reference.layer.SynapseFilter(3.0, step_mode="m")),
                         (layer.Delay(2, step_mode="m"), reference.layer.Delay(2, step_mode="m")),
                         (layer.VotingLayer(3, step_mode="m"), reference.layer.VotingLayer(3, step_mode="m"))):
        torch.testing.assert_close(ours(s), theirs(s))
    c = torch.randint(0, 4, (3, 2, 5)).float()
    ours, theirs = layer.SpikeCountToBinary(3, True), reference.layer.SpikeCountToBinary(3, True)
    torch.testing.assert_close(ours(c), theirs(c))
    torch.testing.assert_close(layer.TemporalBinSum(3, True)(ours(c)), reference.layer.TemporalBinSum(3, True)(theirs(c)))
