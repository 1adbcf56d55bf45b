"""Operation counters and the compute-energy estimate."""
import pytest
import torch
import torch.nn as nn

from spikingjelly_b200.activation_based import functional, layer, neuron
from spikingjelly_b200.activation_based import op_counter as O


def test_rules_on_hand_computed_cases():
    x, w = torch.randn(3, 4), torch.randn(4, 5)
    s = (torch.rand(3, 4) > 0.5).float()
    flop, mac, ac, syn, mem = O.FlopCounter(), O.MACCounter(), O.ACCounter(), O.SynOpCounter(), O.MemoryAccessCounter()
    with O.DispatchCounterMode([flop, mac, ac, syn, mem]):
        torch.mm(x, w)
        torch.mm(s, w)
    assert flop.get_total() == 2 * 3 * 5 * (2 * 4 - 1)
    assert mac.get_total() == 3 * 5 * 4                       # the spike product costs no MAC
    assert syn.get_total() == int(s.sum()) * 5 == ac.get_total()
    assert mem.get_total() == 2 * 4 * (3 * 4 + 4 * 5 + 3 * 5)
    assert O.is_binary_tensor(s) and not O.is_binary_tensor(x) and O.is_binary_tensor(torch.tensor([True]))


def test_counts_are_booked_per_module_and_respect_ignore_lists():
    net = nn.Sequential(layer.Linear(8, 4), neuron.IFNode(), layer.Linear(4, 2))
    c = O.FlopCounter()
    with O.DispatchCounterMode([c]):
        net(torch.rand(5, 8)).sum().backward()
    counts = c.get_counts()
    assert set(counts) >= {"Global", "Sequential", "Sequential.0", "Sequential.2"}
    assert counts["Global"][torch.ops.aten.addmm.default] == counts["Sequential.0"][torch.ops.aten.addmm.default] + counts["Sequential.2"][torch.ops.aten.addmm.default]
    functional.reset_net(net)
    ignoring = O.FlopCounter(extra_ignore_modules=[neuron.IFNode])
    with O.DispatchCounterMode([ignoring]):
        net(torch.rand(5, 8))
    assert "Sequential.1" not in ignoring.get_counts() or not ignoring.get_counts()["Sequential.1"]
    with pytest.raises(NotImplementedError):
        with O.DispatchCounterMode([O.MACCounter()], strict=True):
            torch.rand(3).exp()
    c.reset()
    assert c.get_total() == 0


def test_function_counter_mode_with_custom_rule():
    c = O.BaseCounter(extra_rules={torch.nn.functional.linear: lambda a, k, o: o.numel()})
    with O.FunctionCounterMode([c]):
        torch.nn.functional.linear(torch.rand(2, 3), torch.rand(4, 3))
    assert c.get_total() == 8


def test_energy_estimate_is_dominated_by_accumulates_for_spiking_layers():
    torch.manual_seed(0)
    net = nn.Sequential(layer.Conv2d(2, 4, 3, padding=1), layer.BatchNorm2d(4), neuron.IFNode(), layer.Flatten(), layer.Linear(256, 10))
    spikes = (torch.rand(2, 2, 8, 8) > 0.5).float()
    rep = O.estimate_compute_energy(net, spikes)
    assert rep.counts["mac"] > 0 and rep.counts["synop"] > 0 and rep.counts["ac"] >= rep.counts["synop"]
    assert rep.energy_total_pj == pytest.approx(rep.counts["mac"] * 4.6 + rep.counts["ac"] * 0.9)
    dense = O.estimate_compute_energy(net, torch.rand(2, 2, 8, 8))
    assert dense.counts["mac"] > rep.counts["mac"]            # analog input: the first convolution is all MACs
    cheap = O.estimate_compute_energy(net, spikes, config=O.ComputeEnergyConfig(cost_config=O.ComputeEnergyCostConfig.int8()))
    assert cheap.energy_total_pj < rep.energy_total_pj and "Global" in rep.breakdown_pj
