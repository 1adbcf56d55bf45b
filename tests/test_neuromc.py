"""NeuroMC energy model (role of the reference's ``test/activation_based/op_counter`` NeuroMC cases): counter rules on
hand-computed cases, the report's arithmetic identities, spike-driven against dense cores, the accounting switches,
optimizer modelling, stage handling and unsupported-operator reporting."""
import pytest
import torch
import torch.nn as nn

from spikingjelly_b200.activation_based import functional, layer, neuron, op_counter
from spikingjelly_b200.activation_based.op_counter import neuromc as N
from spikingjelly_b200.activation_based.op_counter.neuromc import core as C


def _count(counter, fn):
    with op_counter.DispatchCounterMode([counter]):
        fn()
    return counter


def test_dense_and_spike_matmul_rules():
    a, b = torch.randn(3, 5), torch.randn(5, 4)
    add = _count(N.NeuroMCAddCounter(), lambda: a @ b)
    mul = _count(N.NeuroMCMulCounter(), lambda: a @ b)
    assert add.get_op_counts() == {"aten.mm.default": 3 * 4 * 4} and mul.get_op_counts() == {"aten.mm.default": 3 * 4 * 5}
    s = torch.tensor([[1.0, 0, 1, 1, 0], [0, 0, 0, 0, 0], [1, 0, 0, 0, 0]])
    add = _count(N.NeuroMCAddCounter(), lambda: s @ b)
    mul = _count(N.NeuroMCMulCounter(), lambda: s @ b)
    # rows with 3, 0 and 1 spikes accumulate 2, 0 and 0 times per output column; no multiplier is used
    assert add.get_total() == 2 * 4 and mul.get_total() == 0
    assert add.get_stage_counts() == {"forward": 8}


def test_convolution_and_elementwise_rules():
    x, w = torch.randn(2, 3, 6, 6), torch.randn(4, 3, 3, 3)
    out_numel = 2 * 4 * 4 * 4
    mul = _count(N.NeuroMCMulCounter(), lambda: torch.nn.functional.conv2d(x, w))
    add = _count(N.NeuroMCAddCounter(), lambda: torch.nn.functional.conv2d(x, w, torch.zeros(4)))
    assert mul.get_total() == out_numel * 27 and add.get_total() == out_numel * 26 + out_numel
    spikes = (torch.rand(2, 3, 6, 6) > 0.5).float()
    assert _count(N.NeuroMCMulCounter(), lambda: torch.nn.functional.conv2d(spikes, w)).get_total() == 0
    hits = torch.nn.functional.conv2d(spikes, torch.ones_like(w))
    assert _count(N.NeuroMCAddCounter(), lambda: torch.nn.functional.conv2d(spikes, w)).get_total() == int((hits - 1).clamp_min(0).sum())
    v = torch.randn(7, 3)
    assert _count(N.NeuroMCCmpCounter(), lambda: v > 0).get_total() == 21
    assert _count(N.NeuroMCMuxCounter(), lambda: torch.where(v > 0, v, torch.zeros_like(v))).get_total() == 21
    assert _count(N.NeuroMCSqrtCounter(), lambda: v.abs().sqrt()).get_total() == 21
    assert _count(N.NeuroMCMulCounter(), lambda: torch.add(v, v, alpha=2.0)).get_total() == 21
    assert _count(N.NeuroMCMulCounter(), lambda: v + v).get_total() == 0
    pool = _count(N.NeuroMCCmpCounter(), lambda: torch.nn.functional.max_pool2d(x, 2))
    assert pool.get_total() == 2 * 3 * 3 * 3 * 3
    pool.reset()
    assert pool.get_total() == 0 and pool.get_op_counts() == {}


def _net():
    net = nn.Sequential(layer.Conv2d(3, 8, 3, padding=1, bias=False), layer.BatchNorm2d(8), neuron.IFNode(),
                        layer.Conv2d(8, 16, 3, padding=1, bias=False), layer.BatchNorm2d(16), neuron.IFNode(), layer.Flatten(),
                        layer.Linear(16 * 8 * 8, 10))
    functional.set_step_mode(net, "m")
    return net


def test_training_step_report_identities():
    torch.manual_seed(0)
    net = _net()
    opt = torch.optim.SGD(net.parameters(), lr=0.1, momentum=0.9, weight_decay=1e-4)
    rep = N.estimate_neuromc_runtime_energy(net, torch.rand(4, 2, 3, 8, 8), target=torch.randn(4, 2, 10), loss_fn=nn.functional.mse_loss, optimizer=opt)
    assert rep.energy_total_pj == pytest.approx(rep.energy_compute_pj + rep.energy_memory_pj)
    assert rep.energy_compute_pj == pytest.approx(rep.energy_mac_pj + rep.energy_extra_compute_pj)
    assert rep.energy_memory_pj == pytest.approx(rep.energy_base_memory_pj + rep.energy_extra_memory_pj)
    for split in (rep.energy_by_stage, rep.energy_by_op, rep.energy_by_core_type, rep.energy_by_process_key):
        assert sum(split.values()) == pytest.approx(rep.energy_total_pj)
    assert set(rep.energy_by_stage) == {"forward", "backward", "optimizer"}
    # the first convolution sees analog pixels (dense core), the second one and the linear layer see spikes
    assert {"ann_fe", "fp_soma", "wg", "ann_we", "bp_grad", "bp_grad_opt"} <= set(rep.energy_by_core_type)
    macs_conv1, macs_conv2, macs_fc = 4 * 2 * 3 * 8 * 64 * 9, 4 * 2 * 8 * 16 * 64 * 9, 4 * 2 * 1024 * 10
    # forward + weight gradient for all three, data gradient for all but the first layer
    assert rep.primitive_counts["totals"]["mac"] == 2 * (macs_conv1 + macs_conv2 + macs_fc) + macs_conv2 + macs_fc
    assert rep.memory_bits_by_level["by_level_dir"]["sram"]["rh2l"] > 0 and "dram" not in rep.memory_bits_by_level["totals"]
    assert len(rep.mapping_summary) == 7 + 9 + 2 and "total" in rep.summary()      # the update: one vector and one matrix bucket
    assert not rep.warnings
    assert all(p.grad is None for p in net.parameters())


def test_spike_input_is_cheaper_than_analog_input():
    torch.manual_seed(1)
    lin = nn.Linear(64, 32, bias=False)
    analog = N.estimate_neuromc_runtime_energy(lin, torch.rand(16, 64) + 0.01)
    spikes = N.estimate_neuromc_runtime_energy(lin, (torch.rand(16, 64) > 0.5).float())
    assert list(analog.energy_by_core_type) == ["ann_fe"] and list(spikes.energy_by_core_type) == ["fp_soma"]
    assert spikes.energy_mac_pj == pytest.approx(16 * 64 * 32 * C.MAC_COST_PJ["fp_soma"])
    assert analog.energy_mac_pj == pytest.approx(16 * 64 * 32 * C.MAC_COST_PJ["ann_fe"])
    assert spikes.energy_total_pj < analog.energy_total_pj
    inst = N.MemoryHierarchyConfig().memory_instances
    per_spike_bit = inst["reg_1b"].r_cost + inst["sram_fp_conv_in_s"].r_cost
    per_word = lambda reg, sram, w=False: (inst[reg].w_cost if w else inst[reg].r_cost) + (inst[sram].w_cost if w else inst[sram].r_cost)
    want = 16 * 64 * per_spike_bit + 64 * 32 * per_word("reg_16b", "sram_fp_conv_in_w") + 16 * 32 * per_word("reg_16b", "sram_fp_conv_out_xi", True)
    assert spikes.energy_base_memory_pj == pytest.approx(want)


def test_weight_tile_is_fetched_once_for_later_tiles():
    lin = nn.Linear(16, 8, bias=False)
    x = (torch.rand(4, 16) > 0.5).float()
    prof = N.NeuroMCEnergyProfiler()
    prof.bind_model(lin)
    with prof:
        with prof.stage("forward_b0_t0"):
            lin(x)
        first = prof.get_report().energy_base_memory_pj
        with prof.stage("forward_b1_t0"):
            lin(x)
        both = prof.get_report().energy_base_memory_pj
        with pytest.raises(RuntimeError):
            with prof.stage("a"):
                with prof.stage("b"):
                    pass
    assert 0 < both - first < first
    with pytest.raises(RuntimeError):
        with prof.stage("late"):
            pass


def test_optimizer_models_and_config_validation():
    lin = nn.Linear(8, 4)
    x, y = torch.rand(2, 8), torch.rand(2, 4)
    plain = N.estimate_neuromc_runtime_energy(lin, x, target=y, loss_fn=nn.functional.mse_loss, optimizer=torch.optim.SGD(lin.parameters(), lr=0.1))
    adam = N.estimate_neuromc_runtime_energy(lin, x, target=y, loss_fn=nn.functional.mse_loss, optimizer=torch.optim.Adam(lin.parameters()))
    assert plain.counts_by_process_key["with_opt"] == {"fragments": 2, "mac": 0, "mux": 0, "add": 36, "mul": 36, "comp": 0, "sqrt": 0}
    # Adam's model carries a scale and a shift vector per vector parameter: 32 weights + 2 * 4
    assert adam.counts_by_process_key["with_opt"]["sqrt"] == 40 and adam.counts_by_process_key["with_opt"]["fragments"] == 1 and adam.energy_by_stage["optimizer"] > plain.energy_by_stage["optimizer"]
    with pytest.raises(ValueError):
        N.estimate_neuromc_runtime_energy(lin, x, optimizer=torch.optim.SGD(lin.parameters(), lr=0.1))
    with pytest.raises(ValueError):
        N.estimate_neuromc_runtime_energy(lin, x, target=y, loss_fn=nn.functional.mse_loss, optimizer=torch.optim.SGD(lin.parameters(), lr=0.1, momentum=0.9, nesterov=True))
    with pytest.raises(ValueError):
        N.estimate_neuromc_runtime_energy(lin, x, target=y, loss_fn=nn.functional.mse_loss, optimizer=torch.optim.RMSprop(lin.parameters()))
    cfg = N.MemoryHierarchyConfig()
    cfg.memory_instances.pop("sram_2MB")
    with pytest.raises(ValueError, match="sram_2MB"):
        cfg.validate()
    with pytest.raises(ValueError):
        N.MemoryHierarchyConfig(technology_nm=7).validate()
    with pytest.raises(ValueError):
        N.NeuroMCEnergyProfiler(core_type="tpu")
    with pytest.raises(ValueError):
        N.estimate_neuromc_runtime_energy(nn.Conv3d(1, 1, 1), torch.rand(1, 1, 2, 2, 2))


def test_operators_without_a_core_are_reported():
    net = nn.Sequential(nn.Linear(8, 8), nn.Softmax(dim=-1))
    rep = N.estimate_neuromc_runtime_energy(net, torch.rand(2, 8))
    assert any("aten._softmax" in w for w in rep.warnings)
    with pytest.raises(RuntimeError, match="no core"):
        N.estimate_neuromc_runtime_energy(net, torch.rand(2, 8), strict=True)


def test_residency_counter_takes_the_hierarchy():
    c = N.NeuroMCMemoryResidencyCounter(config=N.MemoryHierarchyConfig())
    assert c.simulator.capacity_bits["sram"] == 1048576 + 50331648
    _count(c, lambda: torch.randn(4, 4) @ torch.randn(4, 4))
    assert c.get_total() > 0
