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
    assert cheap.energy_total_pj < rep.energy_total_pj and "Global" in rep.per_module_pj and set(rep.breakdown_pj) == {"mac_pj", "ac_pj"}


def test_neuron_state_counter_classifies_state_traffic():
    from spikingjelly_b200.activation_based import functional, layer, neuron
    from spikingjelly_b200.activation_based import op_counter as oc
    torch.manual_seed(0)
    net = torch.nn.Sequential(layer.Linear(8, 16), neuron.LIFNode(tau=2.0), layer.Linear(16, 4), neuron.IFNode())
    functional.set_step_mode(net, "m")
    c = oc.NeuronStateCounter()
    with oc.DispatchCounterMode([c]):
        net(torch.rand(4, 3, 8) * 2)
    m, p = c.get_metric_counts()["Global"], c.get_projection_counts()["Global"]
    # LIF: (x - v) , * 1/tau, + v, reset ... per element and step; the IF neuron has no multiply except the reset
    assert m["state_muls"] == 4 * 3 * 16 * 2 and m["state_comps"] == 4 * 3 * 16
    assert m["spike_triggered_ops"] == m["state_reset_ops"] > 0 and m["timestep_dense_ops"] > 0
    assert p["state_acc_like"] == m["state_adds"] + m["state_comps"] + m["state_select_ops"] + m["state_nonlinear_ops"]
    assert p["potential_buffer_bytes"] == 3 * 16 * 4 and p["read_potential"] == m["state_reads"]
    assert set(c.get_metric_counts()) >= {"Global"} and c.get_extra_counts() == c.get_projection_counts()
    c.reset()
    assert c.get_metric_counts() == {}
    native = neuron.LIFNode(step_mode="m")
    native._backend = "cuda"                                         # kernels hide the state arithmetic from ATen
    with pytest.warns(RuntimeWarning):
        with oc.DispatchCounterMode([c]):
            try:
                native(torch.rand(2, 4))
            except Exception:
                pass
    with pytest.raises(TypeError):
        oc.NeuronStateCounter(extra_state_rules={neuron.IFNode: 3})


def test_lemaire_energy_report_is_consistent():
    from spikingjelly_b200.activation_based import functional, layer, neuron
    from spikingjelly_b200.activation_based import op_counter as oc
    torch.manual_seed(0)
    net = torch.nn.Sequential(layer.Conv2d(2, 4, 3, padding=1), neuron.LIFNode(), layer.Flatten(), layer.Linear(4 * 36, 16), neuron.IFNode(),
                              layer.Linear(16, 4))
    functional.set_step_mode(net, "m")
    x = (torch.rand(4, 3, 2, 6, 6) > 0.6).float()
    r = oc.estimate_lemaire_energy(net, x)
    b = r.breakdown_pj
    assert abs(r.total_pj - (b["ops_pj"] + b["addressing_pj"] + b["memory_pj"])) < 1e-6
    assert abs(b["memory_pj"] - (b["inout_pj"] + b["params_pj"] + b["potential_pj"])) < 1e-6
    spikes_in = int(x.count_nonzero())
    assert r.counts["read_in_bytes"] >= spikes_in * 4 and r.counts["mac"] == 0 and r.counts["mac_addr"] == 2 * spikes_in
    cost = oc.LemaireEnergyCostConfig()
    assert cost.memory_cost_pj(0) == 0 and abs(cost.memory_cost_pj(8192) - 2.5) < 1e-9 and abs(cost.memory_cost_pj(1 << 30) - 25.0) < 1e-9
    assert abs(cost.memory_cost_pj(20 * 1024) - (2.5 + 2.5 * 12 / 24)) < 1e-9
    with pytest.raises(ValueError):
        oc.LemaireEnergyCostConfig(memory_breakpoints=((0.0, 0.0), (1.0, 1.0), (1.0, 2.0), (3.0, 3.0)))
    dense = oc.estimate_lemaire_energy(torch.nn.Sequential(torch.nn.Linear(8, 8), torch.nn.ReLU(), torch.nn.Linear(8, 2)), torch.randn(5, 8))
    assert dense.counts["mac"] == 5 * 8 * 8 + 5 * 8 * 2 and dense.counts["synop"] == 0 and dense.counts["read_potential_bytes"] == 0


def test_memory_residency_hierarchy():
    from spikingjelly_b200.activation_based import op_counter as oc
    sim = oc.MemoryResidencySimulator(capacity_bits={"reg": 64 * 32, "sram": 256 * 32})
    a, b, big = torch.zeros(32), torch.zeros(48), torch.zeros(512)
    sim.on_tensor_read(a, "op")                          # dram -> sram -> reg
    assert sim.get_move_bits_by_edge() == {"dram->sram": 1024, "sram->reg": 1024}
    assert sim.get_level_rw_bits()["dram"] == {"read_bits": 1024, "write_bits": 0, "total_bits": 1024}
    sim.on_tensor_read(a, "op")                          # register hit
    assert sim.get_level_rw_bits()["reg"]["read_bits"] == 2048 and sim.get_move_bits_by_edge()["sram->reg"] == 1024
    sim.on_tensor_read(b, "op")                          # evicts a from the register file back to SRAM (already resident there)
    assert "reg->sram" in sim.get_move_bits_by_edge() and list(sim.reg_cache) == [sim._tensor_key(b)]
    sim.on_tensor_read(big, "op")                        # larger than every on-chip level: streamed from DRAM
    assert sim.get_level_rw_bits()["dram"]["read_bits"] == 1024 + 48 * 32 + 512 * 32 and sim._tensor_key(big) not in sim.sram_cache
    sim.on_tensor_write(torch.zeros(8), "op2")           # a small result is born in the register file
    assert sim.get_op_level_rw_bits()["op2"]["reg"]["write_bits"] == 256
    assert sim.usage_bits["reg"] <= 64 * 32 and sim.usage_bits["sram"] <= 256 * 32
    c = oc.MemoryResidencyCounter(capacity_bits={"reg": 4096 * 8, "sram": 64 * 1024 * 8})
    net = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.ReLU(), torch.nn.Linear(32, 4))
    with oc.DispatchCounterMode([c]):
        net(torch.randn(8, 16)).sum().backward()
    levels = c.get_level_bits()
    assert levels["reg"] > 0 and c.get_total() > 0 and sum(c.get_move_bits_by_edge().values()) > 0
    assert "aten.addmm" in next(iter(k for k in c.get_op_level_bits() if "addmm" in k))
    c.reset()
    assert c.get_level_bits() == {}


def _spikesim_net(ab):
    torch.manual_seed(0)
    return torch.nn.Sequential(
        ab.layer.Conv2d(3, 70, 3, padding=1, bias=False), ab.neuron.IFNode(),
        ab.layer.Conv2d(70, 130, 3, stride=2, padding=1, bias=False), ab.neuron.LIFNode(),
        ab.layer.Conv2d(130, 20, 1, bias=False)).eval()


@pytest.mark.parametrize("mode", ["dense", "event"])
def test_spikesim_energy_equals_reference(mode):
    import importlib, sys
    from pathlib import Path
    import spikingjelly_b200.activation_based as ours_ab
    from spikingjelly_b200.activation_based.op_counter import spikesim as ours
    net = _spikesim_net(ours_ab)
    x = torch.rand(2, 3, 12, 12)
    cfg = ours.SpikeSimEnergyConfig(activity_mode=mode, xbar_size=64)
    rep = ours.estimate_spikesim_event_energy(net, x, config=cfg)
    assert rep.counts["stage_count"] == 3 and rep.energy_total_pj > 0
    # dense PE cycles by hand: ceil(Cin/64) * ceil(Cout/64) * sites
    assert rep.counts["dense_pe_cycle_count"] == 1 * 2 * 2 * 144 + 2 * 3 * 2 * 36 + 3 * 1 * 2 * 36
    if mode == "event":
        st = rep.event_stats_by_stage["1" if "1" in rep.event_stats_by_stage else list(rep.event_stats_by_stage)[1]]
        assert st["active_row_count"] <= st["dense_row_count"]
    ref_dir = Path(__file__).resolve().parents[1] / "baseline" / "_ref"
    if not (ref_dir / "spikingjelly").exists():
        pytest.skip("reference package not installed under baseline/_ref")
    sys.path.insert(0, str(ref_dir))
    try:
        ref_ab = importlib.import_module("spikingjelly.activation_based")
        ref = importlib.import_module("spikingjelly.activation_based.op_counter.spikesim")
        importlib.import_module("spikingjelly.activation_based.layer"); importlib.import_module("spikingjelly.activation_based.neuron")
    finally:
        sys.path.remove(str(ref_dir))
    net_r = _spikesim_net(ref_ab)
    net_r.load_state_dict(net.state_dict())
    rep_r = ref.estimate_spikesim_event_energy(net_r, x, config=ref.SpikeSimEnergyConfig(activity_mode=mode, xbar_size=64))
    assert rep.energy_total_pj == pytest.approx(rep_r.energy_total_pj, rel=1e-9)
    assert rep.counts == rep_r.counts
    for stage, e in rep_r.energy_by_stage.items():
        assert rep.energy_by_stage[stage] == pytest.approx(e, rel=1e-9)
    for k, v in rep_r.breakdown_pj.items():
        assert rep.breakdown_pj[k] == pytest.approx(v, rel=1e-9)
