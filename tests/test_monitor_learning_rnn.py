"""Monitors, STDP learners, spiking RNNs and the conv-BN graph rewrites (host-side)."""
import time

import pytest
import torch
import torch.nn as nn

from spikingjelly_b200.activation_based import functional, layer, learning, monitor, neuron, rnn, surrogate
from spikingjelly_b200.activation_based.functional import conv_bn_fusion


def test_monitors_record_per_layer_and_can_be_paused():
    net = nn.Sequential(layer.Linear(4, 8), neuron.IFNode(), layer.Linear(8, 2), neuron.IFNode())
    out = monitor.OutputMonitor(net, neuron.IFNode, lambda s: float(s.detach().mean()))
    inp = monitor.InputMonitor(net, layer.Linear)
    v = monitor.AttributeMonitor("v", False, net, neuron.IFNode)
    gi, go = monitor.GradInputMonitor(net, neuron.IFNode), monitor.GradOutputMonitor(net, neuron.IFNode)
    x = torch.rand(3, 4, requires_grad=True)
    net(x).sum().backward()
    assert out.monitored_layers == ["1", "3"] and len(out.records) == 2 and len(out["3"]) == 1
    assert inp["0"][0].shape == (3, 4) and v["1"][0].shape == (3, 8)
    assert len(gi.records) == 2 and go["3"][0].shape == (3, 2)       # backward visits layer 3 first
    assert go.name_records_index["3"] == [0]
    out.disable(); net(x)
    assert len(out.records) == 2 and not out.is_enable()
    out.enable(); out.clear_recorded_data()
    assert out.records == [] and out.name_records_index == {"1": [], "3": []}
    out.remove_hooks(); net(x)
    assert out.records == []
    with pytest.raises(ValueError):
        out[1.5]


def test_gpu_monitor_thread_uses_injected_sampler():
    seen = []
    gm = monitor.GPUMonitor(None, (0, 1), 0.005, sampler=lambda: seen.append(1) or [(10, 100), (20, 200)])
    time.sleep(0.05)
    gm.stop(); gm.join(1.0)
    assert gm.step >= 1 and seen and not gm.is_alive()


def _manual_stdp(x_seq, s_seq, w, tau_pre, tau_post):
    tr_pre, tr_post, dw = torch.zeros_like(x_seq[0]), torch.zeros_like(s_seq[0]), torch.zeros_like(w)
    for x, s in zip(x_seq, s_seq):
        tr_pre = tr_pre - tr_pre / tau_pre + x
        tr_post = tr_post - tr_post / tau_post + s
        dw += w * (s.t() @ tr_pre) - w * (tr_post.t() @ x)      # default f_pre / f_post: the weight itself
    return dw


@pytest.mark.parametrize("step_mode", ["s", "m"])
def test_stdp_learner_matches_the_trace_equations(step_mode):
    torch.manual_seed(0)
    net = nn.Sequential(layer.Linear(6, 4, bias=False), neuron.IFNode(v_threshold=0.4))
    functional.set_step_mode(net, step_mode)
    learner = learning.STDPLearner(step_mode, net[0], net[1], 2.0, 3.0)
    x = (torch.rand(5, 3, 6) > 0.4).float()
    with torch.no_grad():
        out = net(x) if step_mode == "m" else torch.stack([net(x[t]) for t in range(5)])
    learner.step(on_grad=True)
    expect = _manual_stdp(x, out, net[0].weight.data, 2.0, 3.0)
    assert torch.allclose(net[0].weight.grad, -expect, atol=1e-5)
    learner.reset()
    assert learner.trace_pre is None and learner.in_spike_monitor.records == []


def test_stdp_conv_and_reward_learners():
    torch.manual_seed(1)
    net = nn.Sequential(layer.Conv2d(2, 3, 3, padding=1, bias=False), neuron.IFNode(v_threshold=0.3))
    learner = learning.STDPLearner("s", net[0], net[1], 2.0, 2.0, f_pre=lambda w: w.abs())
    with torch.no_grad():
        for _ in range(3):
            net((torch.rand(2, 2, 6, 6) > 0.5).float())
    dw = learner.step(on_grad=False, scale=0.5)
    assert dw.shape == net[0].weight.shape and net[0].weight.grad is None and dw.abs().sum() > 0
    with pytest.raises(NotImplementedError):
        learning.stdp_conv2d_single_step(nn.Conv2d(2, 2, 3, dilation=2), torch.zeros(1, 2, 8, 8), torch.zeros(1, 2, 4, 4),
                                         None, None, 2.0, 2.0)
    fc = nn.Sequential(layer.Linear(5, 3, bias=False), neuron.IFNode(v_threshold=0.2))
    m = learning.MSTDPLearner("s", 2, fc[0], fc[1], 2.0, 2.0)
    reward = torch.tensor([1.0, -1.0], requires_grad=True) * 2
    with torch.no_grad():
        for _ in range(3):
            fc((torch.rand(2, 5) > 0.3).float())
    m.step(reward)
    assert fc[0].weight.grad is not None and not fc[0].weight.grad.requires_grad
    with pytest.raises(NotImplementedError):
        learning.MSTDPLearner("m", 2, fc[0], fc[1], 2.0, 2.0).step(reward)
    et = learning.MSTDPETLearner("s", fc[0], fc[1], 2.0, 2.0, 10.0)
    with torch.no_grad():
        for _ in range(3):
            fc((torch.rand(5) > 0.3).float())
    assert et.step(0.5, on_grad=False).shape == (3, 5) and et.trace_e is not None


@pytest.mark.parametrize("cls,n_states", [(rnn.SpikingLSTM, 2), (rnn.SpikingGRU, 1), (rnn.SpikingVanillaRNN, 1)])
@pytest.mark.parametrize("bidirectional", [False, True])
def test_stacked_rnn_equals_cell_by_cell_evaluation(cls, n_states, bidirectional):
    torch.manual_seed(0)
    net = cls(5, 7, 2, bidirectional=bidirectional).eval()
    x = torch.randn(6, 3, 5)
    y, states = net(x)
    dirs = 2 if bidirectional else 1
    assert y.shape == (6, 3, 7 * dirs)
    # reference evaluation through the public cell-level helpers
    cur = x
    for l in range(2):
        z = torch.zeros(3, 7) if n_states == 1 else torch.zeros(2, 3, 7)
        if bidirectional:
            cur, _, _ = rnn.bidirectional_rnn_cell_forward(net.cells[l], net.cells_reverse[l], cur, z, z.clone())
        else:
            cur, _ = rnn.directional_rnn_cell_forward(net.cells[l], cur, z)
    assert torch.allclose(cur, y, atol=1e-6)
    last = states[0] if n_states == 2 else states
    assert last.shape == (2 * dirs, 3, 7) and torch.allclose(last[1], y[-1, :, :7], atol=1e-6)
    y2, _ = net(x, states)                                   # accepts its own final states
    assert y2.shape == y.shape
    with pytest.raises((TypeError, ValueError)):
        net(x, [1, 2])
    y.sum().backward()
    assert all(p.grad is not None for p in net.parameters())


def test_rnn_dropout_masks():
    torch.manual_seed(0)
    net = rnn.SpikingVanillaRNN(4, 16, 3, dropout_p=0.5, invariant_dropout_mask=True, surrogate_function=surrogate.Erf(spiking=False))
    net.train()
    assert net(torch.randn(5, 2, 4))[0].shape == (5, 2, 16)


def test_conv_bn_rewrites():
    torch.manual_seed(0)
    net = nn.Sequential(layer.Conv2d(3, 8, 3, padding=1, bias=False), layer.BatchNorm2d(8), neuron.IFNode(),
                        layer.Conv2d(8, 8, 3, padding=1), layer.BatchNorm2d(8), neuron.IFNode())
    functional.set_step_mode(net, "m")
    x = torch.rand(4, 2, 3, 8, 8)
    net.train()
    with pytest.raises(ValueError):
        conv_bn_fusion.fuse_conv_bn_eval_modules(net)
    y0 = net(x); functional.reset_net(net)
    for m in net.modules():
        if isinstance(m, nn.BatchNorm2d):
            m.reset_running_stats()
    packed = conv_bn_fusion.pack_conv_bn_train_modules(net)
    y1 = packed(x); functional.reset_net(net)
    assert torch.allclose(y0, y1) and "1" not in dict(packed.named_modules())
    net.eval()
    with pytest.raises(ValueError):
        conv_bn_fusion.pack_conv_bn_train_modules(net)
    y2 = net(x); functional.reset_net(net)
    fused = conv_bn_fusion.fuse_conv_bn_eval_modules(net)
    assert torch.allclose(fused(x), y2, atol=1e-5)
    assert not any(isinstance(m, nn.BatchNorm2d) for m in fused.modules())
