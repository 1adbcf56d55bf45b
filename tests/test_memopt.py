"""Compressed-input gradient checkpointing and its automatic placement (host-side, no GPU)."""
import copy
import pickle

import pytest
import torch
import torch.nn as nn

from spikingjelly_b200.activation_based import functional, layer, memopt, neuron, surrogate
from spikingjelly_b200.activation_based.memopt import pipeline
from spikingjelly_b200.activation_based.profiler import (LayerWiseFPCUDATimeProfiler, LayerWiseMemoryProfiler,
                                                         SavedActivationMeter)


class Block(nn.Sequential):
    def __init__(self, c):
        super().__init__(layer.Linear(c, c, step_mode="m"), neuron.LIFNode(step_mode="m", surrogate_function=surrogate.ATan()))


class Splittable(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.a, self.b = Block(c), Block(c)

    def forward(self, x):
        return self.b(self.a(x))

    def __spatial_split__(self):
        return [self.a, self.b]


class Net(nn.Module):
    def __init__(self, c=16, block=Block, n=3):
        super().__init__()
        self.inp = nn.Sequential(layer.Linear(8, c, step_mode="m"), neuron.IFNode(step_mode="m"))
        self.blocks = nn.Sequential(*[block(c) for _ in range(n)])
        self.head = layer.Linear(c, 4, step_mode="m")

    def forward(self, x):
        return self.head(self.blocks(self.inp(x)))


def _grads(net, x):
    functional.reset_net(net)
    net.zero_grad()
    y = net(x)
    y.sum().backward()
    return y.detach(), [p.grad.clone() for p in net.parameters()]


@pytest.mark.parametrize("cls", [memopt.NullSpikeCompressor, memopt.BooleanSpikeCompressor, memopt.Uint8SpikeCompressor,
                                 memopt.BitSpikeCompressor, memopt.SparseSpikeCompressor])
@pytest.mark.parametrize("shape", [(5, 7, 3), (8,), (3, 13)])
def test_compressor_round_trip(cls, shape):
    c = cls()
    s = (torch.rand(shape) > 0.6).float()
    packed = c.compress(s)
    assert torch.equal(c.decompress(packed, tuple(shape)), s)
    assert torch.equal(c.decompress(packed, torch.Size(shape)), s)
    if cls is memopt.BitSpikeCompressor:
        assert packed.dtype == torch.uint8 and packed.numel() == (s.numel() + 7) // 8


def test_bit_layout_is_little_endian_within_a_byte():
    s = torch.zeros(16)
    s[0] = s[3] = s[9] = 1
    assert memopt.bit_spike_compress(s).tolist() == [0b00001001, 0b00000010]


def test_in_gc_first_forward_flag_and_autocast_query():
    seen = []

    def f(x):
        seen.append(memopt.in_gc_1st_forward())
        return x * 2

    x = torch.rand(3, requires_grad=True)
    memopt.input_compressed_gc(f, memopt.NullSpikeCompressor(), x).sum().backward()
    assert seen == [True, False] and not memopt.in_gc_1st_forward()
    dev, dt, on = memopt.query_autocast()
    assert on is False
    with torch.autocast("cpu", torch.bfloat16):
        assert memopt.query_autocast() == ("cpu", torch.bfloat16, True)


def test_input_compressed_gc_matches_plain_autograd_with_dropout():
    lin = nn.Linear(6, 6)
    drop = nn.Dropout(0.5)

    def f(x, scale):
        return drop(lin(x)) * scale

    x = (torch.rand(4, 6) > 0.5).float()
    scale = torch.rand(6, requires_grad=True)
    torch.manual_seed(3)
    y0 = f(x, scale)
    y0.sum().backward()
    g0, s0 = lin.weight.grad.clone(), scale.grad.clone()
    lin.zero_grad(); scale.grad = None
    torch.manual_seed(3)
    y1 = memopt.to_gc_function(memopt.BitSpikeCompressor(), f)(x, scale)
    y1.sum().backward()
    assert torch.equal(y0, y1) and torch.allclose(g0, lin.weight.grad) and torch.allclose(s0, scale.grad)


def test_gc_container_stateful_and_pickle():
    torch.manual_seed(0)
    ref = Block(8)
    gc = memopt.GCContainer(memopt.BitSpikeCompressor(), *copy.deepcopy(ref))
    x = (torch.rand(4, 2, 8) > 0.5).float()
    # two consecutive calls without reset: the membrane potential must carry over through the container
    for net in (ref, gc):
        functional.reset_net(net)
    y_ref = torch.cat([ref(x), ref(x)])
    y_gc = torch.cat([gc(x), gc(x)])
    assert torch.equal(y_ref, y_gc)
    y_ref.sum().backward(); y_gc.sum().backward()
    for p, q in zip(ref.parameters(), gc.parameters()):
        assert torch.allclose(p.grad, q.grad, atol=1e-6)
    clone = pickle.loads(pickle.dumps(gc))
    functional.reset_net(clone); functional.reset_net(gc)
    assert torch.equal(clone(x), gc(x))
    functional.reset_net(gc)
    assert isinstance(copy.deepcopy(gc), memopt.GCContainer)


@pytest.mark.parametrize("n_chunk", [1, 2, 3, 16])
def test_tcgc_container_matches_unchunked(n_chunk, caplog):
    torch.manual_seed(1)
    ref = Net()
    tc = copy.deepcopy(ref)
    tc.blocks = memopt.TCGCContainer(memopt.BitSpikeCompressor(), *tc.blocks, n_chunk=n_chunk)
    x = torch.rand(6, 3, 8)
    y0, g0 = _grads(ref, x)
    y1, g1 = _grads(tc, x)
    assert torch.allclose(y0, y1, atol=1e-6)
    for a, b in zip(g0, g1):
        assert torch.allclose(a, b, atol=1e-5)


def test_tcgc_multiple_inputs_and_outputs():
    class Two(nn.Module):
        n_seq_inputs, n_outputs = 2, 2

        def __init__(self):
            super().__init__()
            self.lif = neuron.LIFNode(step_mode="m")

        def forward(self, a, b, gain):
            s = self.lif(a + b * gain)
            return s, a - b

    torch.manual_seed(0)
    a, b = torch.rand(6, 2, 5, requires_grad=True), torch.rand(6, 2, 5, requires_grad=True)
    gain = torch.tensor(1.5, requires_grad=True)
    plain = Two()
    s0, d0 = plain(a, b, gain)
    (s0.sum() + d0.sum()).backward()
    ga, gg = a.grad.clone(), gain.grad.clone()
    a.grad = b.grad = gain.grad = None
    box = memopt.TCGCContainer(None, Two(), n_chunk=3, n_seq_inputs=2, n_outputs=2)
    s1, d1 = box(a, b, gain)
    (s1.sum() + d1.sum()).backward()
    assert torch.equal(s0, s1) and torch.allclose(d0, d1)
    assert torch.allclose(ga, a.grad, atol=1e-6) and torch.allclose(gg, gain.grad, atol=1e-5)


def test_saved_activation_meter_sees_checkpointing():
    torch.manual_seed(0)
    plain, wrapped = Net(c=64), Net(c=64)
    wrapped.blocks = nn.Sequential(*[memopt.GCContainer(memopt.BitSpikeCompressor(), b) for b in wrapped.blocks])
    x = torch.rand(8, 4, 8)

    def peak(net):
        with SavedActivationMeter((net,)) as m:
            net(x).sum().backward()
            functional.reset_net(net)
            return m.peak(), m.current()

    p0, live0 = peak(plain)
    p1, live1 = peak(wrapped)
    assert live0 == 0 and live1 == 0          # everything released after backward
    assert p1 < p0


def test_layerwise_profilers_on_host(tmp_path):
    net = Net()
    x = torch.rand(4, 2, 8)
    with LayerWiseMemoryProfiler((net,), ("net",), ("submodules",), (Block,), log_path=tmp_path / "m.txt",
                                 data_path=tmp_path / "m.pt", device="cpu") as prof:
        net(x).sum().backward()
        rows = prof.export()
    assert len(rows) == 3 and all(r[0].startswith("net's blocks.") for r in rows)
    assert all(r[4] > 0 for r in rows)        # forward saved something
    assert (tmp_path / "m.txt").exists() and (tmp_path / "m.pt").exists()
    functional.reset_net(net)
    with torch.no_grad(), LayerWiseFPCUDATimeProfiler((net,), instances=(nn.Sequential,), warmup=1, log_path=tmp_path / "t.txt") as prof:
        for _ in range(3):
            net(x); functional.reset_net(net)
        table = prof.export()
    assert {n for n, _ in table} == {"net0's inp", "net0's blocks"}


def test_resolve_device_validates_local_rank(monkeypatch):
    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    monkeypatch.setattr(torch.cuda, "device_count", lambda: 2)
    monkeypatch.setenv("LOCAL_RANK", "abc")
    with pytest.raises(ValueError, match="LOCAL_RANK must be an integer"):
        memopt.resolve_device()
    monkeypatch.setenv("LOCAL_RANK", "5")
    with pytest.raises(ValueError, match=r"in \[0, 2\)"):
        memopt.resolve_device()
    monkeypatch.setenv("LOCAL_RANK", "1")
    assert memopt.resolve_device() == "cuda:1"


def test_probe_binary_inputs_and_random_like():
    net = Net()
    x = torch.rand(4, 2, 8)
    verdict = pipeline._probe_binary_inputs(net, tuple(net.blocks), (x,))
    assert all(verdict.values())               # blocks see IF/LIF spikes
    verdict = pipeline._probe_binary_inputs(net, (net.inp,), (x,))
    assert verdict[net.inp] is False
    r = pipeline._random_like((torch.zeros(3, dtype=torch.bool), torch.zeros(3, dtype=torch.int64), 5))
    assert r[0].dtype == torch.bool and r[1].dtype == torch.int64 and r[2] == 5


def test_apply_gc_picks_compressors_and_budgets():
    x = torch.rand(4, 2, 8)
    net, info = memopt.apply_gc(Net(), Block, (x,), device="cpu", return_summary=True)
    assert info["gc_wrap_count"] == 3 and info["bit_compressor_count"] == 3
    assert all(isinstance(b, memopt.GCContainer) and isinstance(b.x_compressor, memopt.BitSpikeCompressor) for b in net.blocks)
    net, info = memopt.apply_gc(Net(), Block, (x,), compress_x=False, device="cpu", return_summary=True)
    assert info["null_compressor_count"] == 3
    net, info = memopt.apply_gc(Net(n=4), Block, (x,), device="cpu", checkpoint_budget="speed", return_summary=True)
    assert info["gc_selected_count"] == 2 and info["gc_wrap_count"] == 2 and info["gc_selection_policy"] == "largest_input_activations"
    net, info = memopt.apply_gc(Net(n=4), Block, None, device="cpu", max_gc_wrapped_modules=1, checkpoint_budget="memory", return_summary=True)
    assert info["gc_selection_policy"] == "fallback_module_order" and info["gc_selected_modules"] == ["blocks.0"]
    manual = Net()
    manual.blocks[1].x_compressor = "Uint8SpikeCompressor"
    net, info = memopt.apply_gc(manual, Block, (x,), device="cpu", return_summary=True)
    assert info["manual_compressor_count"] == 1 and isinstance(net.blocks[1].x_compressor, memopt.Uint8SpikeCompressor)
    with pytest.raises(ValueError, match="Unknown compressor spec"):
        bad = Net(); bad.blocks[0].x_compressor = "NoSuchCompressor"
        memopt.apply_gc(bad, Block, (x,), device="cpu")


def test_memory_optimization_option_resolution():
    with pytest.raises(ValueError, match="dummy_input must be provided"):
        memopt.memory_optimization(Net(), Block, None, level=2)
    with pytest.raises(ValueError, match="Unsupported memopt profile"):
        memopt.memory_optimization(Net(), Block, None, profile="nope")
    with pytest.raises(ValueError, match="Unsupported prefer"):
        memopt.memory_optimization(Net(), Block, None, prefer="nope")
    net, s = memopt.memory_optimization(Net(), Block, None, profile="balanced", return_summary=True)
    assert s.requested_level == 2 and s.applied_level == 1 and "fallback:level>1_requires_dummy_input" in s.notes
    net, s = memopt.memory_optimization(Net(n=4), Block, None, prefer="speed", return_summary=True)
    assert s.profile == "safe" and s.checkpoint_budget == "speed" and s.gc_wrap_count == 2
    assert "prefer:profile=safe" in s.notes and s.recommendation.startswith("Current settings favor training speed")
    net, s = memopt.memory_optimization(Net(), Block, None, level=0, return_summary=True)
    assert s.gc_container_count == 0 and s.applied_steps == []


def test_memory_optimization_levels_reduce_saved_activations():
    torch.manual_seed(0)
    x = torch.rand(8, 4, 8)
    base = Net(c=64, block=Splittable, n=2)
    bench = pipeline._Bench((x,), "cpu", warmup=False)
    p0 = bench.peak(base)
    y0, g0 = _grads(copy.deepcopy(base), x)

    net1, s1 = memopt.memory_optimization(copy.deepcopy(base), Splittable, (x,), level=1, return_summary=True)
    p1 = bench.peak(net1)
    assert s1.gc_wrap_count == 2 and p1 < p0

    net2, s2 = memopt.memory_optimization(copy.deepcopy(base), Splittable, (x,), level=2, return_summary=True)
    assert "level2_spatial_split" in s2.applied_steps
    p2 = bench.peak(net2)
    assert p2 <= p1 and s2.gc_container_count == 2 + s2.spatial_split_count

    net3, s3 = memopt.memory_optimization(copy.deepcopy(base), Splittable, (x,), level=3, max_split_rounds=2, return_summary=True)
    assert "level3_temporal_split" in s3.applied_steps
    assert bench.peak(net3) <= p2 and s3.tcgc_container_count == s3.temporal_split_count or s3.temporal_split_count >= 0

    net4, s4 = memopt.memory_optimization(copy.deepcopy(base), Splittable, (x,), level=4, max_split_rounds=1, return_summary=True)
    assert "level4_greedy_unwrap" in s4.applied_steps
    for net in (net1, net2, net3, net4):
        y, g = _grads(net, x)
        assert torch.allclose(y, y0, atol=1e-5)
        for a, b in zip(g, g0):
            assert torch.allclose(a, b, atol=1e-4)


def test_temporal_split_refuses_parallel_neurons():
    box = memopt.GCContainer(None, neuron.PSN(T=4))
    assert pipeline._split_temporally(box) is None
    box = memopt.GCContainer(None, Block(4))
    t = pipeline._split_temporally(box, 2)
    assert isinstance(t, memopt.TCGCContainer) and t.n_chunk == 2
    assert pipeline._split_temporally(t, 2).n_chunk == 4
    assert pipeline._unwrap(box) is box[0] or isinstance(pipeline._unwrap(box), nn.Module)
    m, parent, name = memopt.get_module_and_parent(Net(), "net's blocks.1")
    assert name == "1" and isinstance(m, Block)
