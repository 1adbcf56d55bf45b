"""ANN-to-SNN conversion: calibration modules, rate coding (layer- and channel-wise), exact
temporal-difference conversion, QCFS encoding, delayed read-out."""
import copy

import pytest
import torch
import torch.nn as nn

from spikingjelly_b200.activation_based import ann2snn as A
from spikingjelly_b200.activation_based import functional, neuron
from spikingjelly_b200.activation_based.ann2snn import operators as ops
from spikingjelly_b200.activation_based.ann2snn.modules import _safe_quantile
from spikingjelly_b200.activation_based.ann2snn.sample_models import cifar10_resnet, mnist_cnn


def _calibrated_cnn():
    torch.manual_seed(0)
    ann = mnist_cnn.CNN().eval()
    for m in ann.modules():
        if isinstance(m, nn.BatchNorm2d):
            m.running_mean.normal_(0, 0.1)
            m.running_var.uniform_(0.5, 1.5)
    return ann, [(torch.rand(8, 1, 28, 28), torch.zeros(8)) for _ in range(3)]


def test_quantile_and_voltage_hook_modes():
    x = torch.arange(101.0)
    assert float(_safe_quantile(x, 0.5)) == 50.0 and float(_safe_quantile(x, 0.995)) == pytest.approx(99.5)
    assert torch.allclose(_safe_quantile(torch.stack([x, 2 * x]), 0.25, dim=1), torch.tensor([25.0, 50.0]))
    h = A.VoltageHook(momentum=0.5, mode="Max").train()
    h(torch.tensor([[1.0, 4.0]])); h(torch.tensor([[2.0, 8.0]]))
    assert float(h.scale) == 6.0                      # first batch copies, second averages
    h.eval(); h(torch.tensor([[100.0]]))
    assert float(h.scale) == 6.0
    assert float(A.VoltageHook(mode=0.5).train()(torch.tensor([[4.0]])) .max()) == 4.0
    with pytest.raises(NotImplementedError):
        A.VoltageHook(mode="median").train()(torch.ones(2, 2))
    s = A.ChannelVoltageScaler(torch.tensor([1.0, 2.0]), channel_dim=1, step_mode="m")
    assert torch.equal(s(torch.ones(3, 2, 2, 4))[0, 0, :, 0], torch.tensor([1.0, 2.0]))
    with pytest.raises(ValueError):
        A.ChannelVoltageScaler(torch.tensor([1.0, -2.0]))
    with pytest.raises(ValueError):
        A.NeuronFactory(v_threshold=-1.0)
    with pytest.raises(TypeError):
        A.NeuronFactory(neuron.IFNode, v_threshold=1.0, **{"v_reset": 0.0, "v_threshold": 2.0})


@pytest.mark.parametrize("kw", [dict(mode="Max"), dict(mode="99.9%"), dict(mode=0.8), dict(mode="Max", channel_wise=True),
                                dict(mode="Max", channel_wise=True, half_threshold=True)])
def test_rate_coding_approaches_the_ann_with_more_steps(kw):
    ann, data = _calibrated_cnn()
    snn = A.Converter(A.RateCodingRecipe(data, **kw)).convert(copy.deepcopy(ann))
    assert not any(isinstance(m, (nn.ReLU, nn.BatchNorm2d)) for m in snn.modules())
    assert sum(isinstance(m, neuron.BaseNode) or type(m).__name__.endswith("IFNode") for m in snn.modules()) == 4
    x = data[0][0]
    with torch.no_grad():
        ref = ann(x)

        def err(T):
            functional.reset_net(snn)
            return float((sum(snn(x) for _ in range(T)) / T - ref).abs().mean())
        e8, e64 = err(8), err(64)
        assert e64 < e8 and e64 < 0.05, (e8, e64)
        functional.reset_net(snn)
        single = torch.stack([snn(x) for _ in range(8)])
        functional.reset_net(snn)
        functional.set_step_mode(snn, "m")
        assert torch.allclose(snn(x.unsqueeze(0).repeat(8, 1, 1, 1, 1)), single, atol=1e-5)


def test_rate_coding_on_a_residual_network_and_converter_errors():
    torch.manual_seed(0)
    ann = cifar10_resnet.ResNet18().eval()
    data = [torch.rand(2, 3, 32, 32)]
    snn = A.Converter(A.RateCodingRecipe(data, mode="99%")).convert(ann)
    assert snn(torch.rand(2, 3, 32, 32)).shape == (2, 10)
    with pytest.raises(ValueError, match="requires parameters"):
        A.Converter("rate_coding")
    with pytest.raises(ValueError, match="Unknown ann2snn conversion recipe"):
        A.Converter("nope")
    with pytest.raises(TypeError):
        A.Converter(A.ModuleConversionRecipe())
    with pytest.raises(TypeError):
        A.ModuleConverter(A.RateCodingRecipe(data))
    with pytest.raises(NotImplementedError):
        A.Converter(A.RateCodingRecipe(data, mode="wrong")).convert(cifar10_resnet.ResNet18())

    class Swap(A.ModuleConversionRecipe):
        def convert_module(self, converter, ann):
            return nn.Sequential(ann, neuron.IFNode())
    was_training = ann.training
    out = A.ModuleConverter(Swap()).convert(ann)
    assert isinstance(out[1], neuron.IFNode) and ann.training == was_training


class _Block(nn.Module):
    def __init__(self):
        super().__init__()
        self.ln1, self.ln2 = nn.LayerNorm(16), nn.LayerNorm(16)
        self.attn = nn.MultiheadAttention(16, 4, batch_first=True)
        self.fc1, self.act, self.fc2 = nn.Linear(16, 32), nn.GELU(), nn.Linear(32, 16)

    def forward(self, x):
        h = self.ln1(x)
        x = x + self.attn(h, h, h)[0]
        return x + self.fc2(self.act(self.fc1(self.ln2(x))))


def test_temporal_difference_conversion_is_exact_for_any_step_count():
    torch.manual_seed(0)
    blk = _Block().eval()
    snn = A.Converter("transformer_td_equivalent").convert(copy.deepcopy(blk))
    assert isinstance(snn.fc1, ops.TDLinear) and isinstance(snn.attn, ops.TDMultiheadAttention) and isinstance(snn.ln1, ops.TDLayerNorm)
    assert list(snn.state_dict().keys()) != [] and snn.fc1.weight is not None
    with torch.no_grad():
        for T in (1, 3, 7):
            xs = torch.randn(T, 2, 5, 16) * 0.3
            functional.reset_net(snn)
            functional.set_step_mode(snn, "m")
            y = snn(xs)
            assert torch.allclose(y.sum(0), blk(xs.sum(0)), atol=1e-5)
            functional.reset_net(snn)
            functional.set_step_mode(snn, "s")
            assert torch.allclose(torch.stack([snn(xs[t]) for t in range(T)]), y, atol=1e-5)
        functional.reset_net(snn)
        functional.set_step_mode(snn, "m")
        xs = torch.randn(6, 2, 5, 16) * 0.3
        whole = snn(xs)
        functional.reset_net(snn)
        assert torch.allclose(torch.cat([snn(xs[:2]), snn(xs[2:])]), whole, atol=1e-5)     # state carries across calls


def test_td_operators_individually():
    torch.manual_seed(1)
    xs = torch.randn(5, 3, 8)
    for op, f in ((ops.TDSoftmax(-1), lambda x: torch.softmax(x, -1)), (ops.TDGELU(), nn.functional.gelu), (ops.TDSiLU(), nn.functional.silu),
                  (ops.TDRMSNorm(8), lambda x: nn.functional.rms_norm(x, (8,)))):
        assert torch.allclose(op(xs).sum(0), f(xs.sum(0)), atol=1e-5)
    a, b = torch.randn(4, 2, 3, 5), torch.randn(4, 2, 5, 6)
    assert torch.allclose(ops.SNNMatrixOperator()(a, b).sum(0), a.sum(0) @ b.sum(0), atol=1e-4)
    assert torch.allclose(ops.SNNElementWiseProduct()(a, a).sum(0), a.sum(0) ** 2, atol=1e-4)
    q = torch.randn(4, 2, 2, 5, 8)
    sdpa = ops.TDScaledDotProductAttention(is_causal=True)
    assert torch.allclose(sdpa(q, q, q).sum(0), nn.functional.scaled_dot_product_attention(q.sum(0), q.sum(0), q.sum(0), is_causal=True), atol=1e-5)
    lin = ops.TDLinear(8, 4)
    y = lin(xs)
    assert torch.allclose(y[1], nn.functional.linear(xs[1], lin.weight), atol=1e-6)           # bias only on the first step
    assert torch.allclose(y.sum(0), nn.functional.linear(xs.sum(0), lin.weight, lin.bias), atol=1e-5)
    with pytest.raises(ValueError):
        ops.TDSoftmax()(torch.randn(5))


def test_qcfs_encoder_and_delay_estimate():
    enc = A.SignedQCFSSequenceEncoder(torch.tensor([0.1, 0.2, 0.05, 0.3]), 8)
    x = torch.randn(5, 4) * 0.5
    seq = enc.encode(x)
    assert seq.shape == (8, 5, 4) and torch.allclose(seq.sum(0), enc.reconstruct(x), atol=1e-6)
    levels = seq / torch.tensor([0.1, 0.2, 0.05, 0.3])
    assert torch.all((levels.round() - levels).abs() < 1e-5) and levels.abs().max() <= 1 + 1e-5
    stats = enc.statistics()
    assert 0 <= stats["boundary_correction_fraction"] <= 1 and stats["spike_value_count"] == 8 * 20
    assert torch.allclose(enc(seq), seq.sum(0).unsqueeze(0) * 0 + enc.encode(seq.sum(0)))
    with pytest.raises(ValueError):
        A.SignedQCFSSequenceEncoder(torch.tensor([0.1, -1.0]), 4)
    ann, data = _calibrated_cnn()
    snn = A.Converter(A.RateCodingRecipe(data)).convert(ann)
    d = A.estimate_delay_start(snn, data, "cpu", 64)
    assert 0 < d < 60
    with pytest.warns(RuntimeWarning):
        assert A.estimate_delay_start(snn, data, "cpu", 6) == 1
    assert A.estimate_delay_start(nn.Linear(2, 2), data, "cpu", 8) == 0


def test_local_threshold_balancing_matches_reference_rule():
    ann, data = _calibrated_cnn()
    ltb = A.Converter(A.LocalThresholdBalancingRecipe(data)).convert(copy.deepcopy(ann))
    names = dict(ltb.named_modules())
    assert any(n.endswith("ltb_spiking_0.if_node") for n in names) and not any(isinstance(m, nn.ReLU) for m in ltb.modules())
    assert all(type(m).__name__ == "HalfThresholdIFNode" for n, m in names.items() if n.endswith("if_node"))
    x = data[0][0]
    with torch.no_grad():
        functional.reset_net(ltb)
        err = float((sum(ltb(x) for _ in range(64)) / 64 - ann(x)).abs().mean())
    assert err < 0.1
    # the observer's update rule on a hand-made case: threshold += 2 * mean(overflow)
    from spikingjelly_b200.activation_based.ann2snn.recipes.local_threshold_balancing import LocalThresholdBalancingHook
    h = LocalThresholdBalancingHook(channel_dim=1)
    out = h(torch.tensor([[1.0, -2.0], [3.0, 4.0]]))
    assert torch.allclose(h.threshold, torch.tensor([4.0, 4.0])) and torch.equal(out, torch.tensor([[1.0, 0.0], [3.0, 4.0]]))
