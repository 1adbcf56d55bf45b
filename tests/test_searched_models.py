"""SNASNet and SpikeDHS: shapes, state-dict key parity and numerical equality with the reference implementation when it
is installed (same weights -> same outputs and gradients), and the surrogate-search stage protocol of SpikeDHS."""
import importlib
import sys
from pathlib import Path

import pytest
import torch

from spikingjelly_b200.activation_based import functional
from spikingjelly_b200.models import snas_net, spike_dhs

ROOT = Path(__file__).resolve().parents[1]


def _ref_module(name):
    ref_dir = ROOT / "baseline" / "_ref"
    if not (ref_dir / "spikingjelly").exists():
        pytest.skip("reference package not installed under baseline/_ref")
    sys.path.insert(0, str(ref_dir))
    try:
        return importlib.import_module(f"spikingjelly.activation_based.model.{name}")
    except Exception as exc:  # pragma: no cover
        pytest.skip(f"reference module not importable: {exc}")
    finally:
        sys.path.remove(str(ref_dir))


CON_FWD = [[0, 1, 2, 3], [0, 0, 4, 2], [0, 0, 0, 3], [0, 0, 0, 0]]
CON_BWD = [[0, 1, 2, 3], [2, 0, 4, 2], [1, 3, 0, 3], [4, 0, 2, 0]]


@pytest.mark.parametrize("celltype,con", [("forward", CON_FWD), ("backward", CON_BWD)])
def test_snasnet_shapes_and_reset(celltype, con):
    torch.manual_seed(0)
    args = snas_net.snasnet_args(dataset="cifar10", timestep=2, celltype=celltype)
    net = snas_net.SNASNet(args, con).eval()
    x = torch.randn(2, 3, 32, 32)
    with torch.no_grad():
        y1 = net(x)
        functional.reset_net(net)
        y2 = net(x)
    assert y1.shape == (2, 10)
    torch.testing.assert_close(y1, y2)           # reset_net + neuron_init restore the initial state


@pytest.mark.parametrize("celltype,con", [("forward", CON_FWD), ("backward", CON_BWD)])
def test_snasnet_equals_reference(celltype, con):
    ref = _ref_module("snas_net")
    torch.manual_seed(0)
    args = snas_net.snasnet_args(dataset="cifar100", timestep=3, celltype=celltype)
    ours = snas_net.SNASNet(args, torch.tensor(con)).train()
    theirs = ref.SNASNet(args, torch.tensor(con)).train()
    assert list(ours.state_dict().keys()) == list(theirs.state_dict().keys())
    theirs.load_state_dict(ours.state_dict())
    x = torch.randn(2, 3, 32, 32)
    torch.manual_seed(1)
    ya = ours(x)
    torch.manual_seed(1)
    yb = theirs(x)
    torch.testing.assert_close(ya, yb, rtol=1e-5, atol=1e-6)
    ya.square().sum().backward()
    yb.square().sum().backward()
    ga = dict(ours.named_parameters())
    for name, p in theirs.named_parameters():
        if p.grad is None:
            assert ga[name].grad is None or float(ga[name].grad.abs().max()) == 0.0
        else:
            torch.testing.assert_close(ga[name].grad, p.grad, rtol=1e-4, atol=1e-6)


def test_dspike_gradient_formula():
    x = torch.linspace(-1, 1, 41, dtype=torch.float64, requires_grad=True)
    sg = spike_dhs.DSpike(alpha=3.0)
    y = sg(x)
    assert torch.equal(y, (x >= 0).to(x.dtype))
    y.sum().backward()
    import math
    expect = 3.0 / (2 * math.tanh(1.5)) / torch.cosh(3.0 * x.detach()) ** 2
    expect[x.detach().abs() > 0.5] = 0
    torch.testing.assert_close(x.grad, expect)


def test_network_layer_to_space():
    sp = spike_dhs.network_layer_to_space([0, 0, 1, 1, 2, 1])
    assert sp.shape == (6, 4, 3) and sp.sum() == 6
    assert sp[0, 0, 0] == 1 and sp[1, 0, 1] == 1 and sp[2, 1, 0] == 1 and sp[4, 2, 0] == 1 and sp[5, 1, 2] == 1


def _small_dhs():
    return spike_dhs.SpikeDHS(3, spike_dhs.spikedhs_args(fea_filter_multiplier=48))


def test_spikedhs_forward_backward_and_search_stage():
    torch.manual_seed(0)
    net = _small_dhs().train()
    net._time_step = 2
    x = torch.randn(2, 3, 32, 32)
    logits, aux = net(x)
    assert logits.shape == (2, 100) and aux is not None and aux.shape == (2, 100)
    (logits.sum() + aux.sum()).backward()
    assert net.feature.stem0.conv_m.weight.grad is not None
    functional.reset_net(net)

    stem = net.feature.stem0
    node = net.feature.cells[0]._ops[0]
    for m in (stem, node):
        m.dgs_init_stage()
    assert stem.is_DGS and torch.equal(stem.conv_s.weight, stem.conv_m.weight)
    assert stem.spike_s.surrogate_function.alpha == pytest.approx(2.8) and stem.spike_b.surrogate_function.alpha == pytest.approx(3.2)
    logits, _ = net(x)
    logits.sum().backward()
    assert stem.dgs_alpha.grad is not None and node.dgs_alpha.grad is not None
    assert stem.spike_m.v_before_spike is not None
    stem.dgs_finish_stage(2)
    node.dgs_finish_stage(0)
    assert not stem.is_DGS and stem.spike_m.surrogate_function.alpha == pytest.approx(3.2)
    assert node.spike_m.surrogate_function.alpha == pytest.approx(2.8)
    functional.reset_net(net)
    net.eval()
    with torch.no_grad():
        logits, aux = net(x)
    assert aux is None and logits.shape == (2, 100)


def test_spikedhs_state_dict_keys_equal_reference():
    ref = _ref_module("spike_dhs")
    import inspect
    if "cuda()" in inspect.getsource(ref.SearchSpikingConv2d_stem.__init__) and not torch.cuda.is_available():
        # the reference places a parameter on "cuda" in its constructor: compare against the names in its source instead
        src = inspect.getsource(ref)
        ours = set(k.split(".")[-2] + "." + k.split(".")[-1] for k in _small_dhs().state_dict().keys())
        for stem in ("conv_m", "conv_b", "conv_s", "bn_m", "bn_b", "bn_s", "conv1_m", "conv2_s", "bn1_b", "bn2_m"):
            assert f"self.{stem} =" in src and any(k.startswith(stem + ".") for k in ours)
        return
    args = spike_dhs.spikedhs_args()
    ours = spike_dhs.SpikeDHS(3, args)
    theirs = ref.SpikeDHS(3, args)
    assert sorted(ours.state_dict().keys()) == sorted(theirs.state_dict().keys())
