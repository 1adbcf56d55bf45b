"""Neuron modules against the installed reference package (``baseline/_ref``) on the CPU: same constructor arguments, same
state dict, same input -> same single-step and multi-step outputs (spikes and every other returned tensor) and the same input
gradient.  Skipped when the reference is not installed."""
import inspect
import sys
import warnings
from pathlib import Path

import pytest
import torch

REF = Path(__file__).resolve().parents[1] / "baseline" / "_ref"
pytestmark = pytest.mark.skipif(not (REF / "spikingjelly").is_dir(), reason="reference package not installed under baseline/_ref")

# constructor arguments for the classes that need some
ARGS = {
    "GatedLIFNode": dict(T=6), "DSRIFNode": dict(T=6), "DSRLIFNode": dict(T=6), "LIAFNode": dict(act=torch.relu, threshold_related=False), "SimpleLIFNode": dict(tau=2.0, decay_input=True),
    "MPBNLIFNode": dict(out_features=8), "NoisyCUBALIFNode": dict(num_node=8), "NoisyNonSpikingIFNode": dict(num_node=8),
    "ILCLIFNode": dict(act_dim=8, dec_pop_dim=1), "ILCIFNode": dict(act_dim=8, dec_pop_dim=1), "ILCCUBALIFNode": dict(act_dim=8, dec_pop_dim=1),
    "PSN": dict(T=6), "MaskedPSN": dict(k=2, T=6), "SlidingPSN": dict(k=2),
}
SKIP = {"BaseNode", "AdaptBaseNode", "SimpleBaseNode", "NonSpikingBaseNode", "MPBNBaseNode", "NoisyBaseNode", "NoisyILCBaseNode", "ILCBaseNode",
        "NoisyNonSpikingBaseNode", "FewSpikeNode", "HGNode", "OutlierAwareThresholdNode", "NoisyILCCUBALIFNode"}


# nodes whose ``forward`` always consumes a whole sequence ``[T, N, ...]`` (they have no ``step_mode``)
SEQUENCE_ONLY = {"PSN", "MaskedPSN", "SlidingPSN", "ILCLIFNode", "ILCIFNode", "ILCCUBALIFNode", "NoisyCUBALIFNode", "NoisyNonSpikingIFNode",
                 "NonSpikingIFNode", "NonSpikingLIFNode"}


def _packages():
    warnings.simplefilter("ignore")
    if str(REF) not in sys.path:
        sys.path.insert(0, str(REF))
    from spikingjelly.activation_based import functional as rf, neuron as rn
    from spikingjelly_b200.activation_based import functional as of, neuron as on
    return (on, of), (rn, rf)


def _names():
    (on, _), (rn, _) = _packages()
    out = []
    for n in sorted(dir(rn)):
        cls = getattr(rn, n)
        if inspect.isclass(cls) and hasattr(on, n) and n not in SKIP and (n.endswith("Node") or n in ARGS):
            out.append(n)
    return out


def _first(y):
    return y[0] if isinstance(y, (tuple, list)) else y


def _flat(y):
    return [t for t in (y if isinstance(y, (tuple, list)) else (y,)) if torch.is_tensor(t)]


@pytest.mark.parametrize("name", _names() if (REF / "spikingjelly").is_dir() else [])
def test_neuron_equals_the_reference(name):
    (on, of), (rn, rf) = _packages()
    kw = ARGS.get(name, {})
    torch.manual_seed(0)
    a = getattr(on, name)(**kw)
    torch.manual_seed(0)
    b = getattr(rn, name)(**kw)
    b.load_state_dict(a.state_dict())
    x0 = torch.rand(6, 3, 8) * 2.2
    if hasattr(a, "reset_noise"):                       # the noise tables come from an unseeded generator: share them
        a.reset_noise(6)
        b.reset_noise(6)
        for k, v in vars(a).items():
            if k.startswith("eps_") and torch.is_tensor(v):
                assert getattr(b, k).shape == v.shape, k
                setattr(b, k, v.clone())
    results = []
    for m, F_ in ((a, of), (b, rf)):
        m.train()
        outs = {}
        if name not in SEQUENCE_ONLY:
            try:
                F_.reset_net(m)
                F_.set_step_mode(m, "s")
                torch.manual_seed(1)
                leaf = x0.clone().requires_grad_(True)
                x = leaf * 1.0                                   # some reference neurons write into views of their input
                steps = [m(x[t]) for t in range(6)]
                y = torch.stack([_first(s) for s in steps])
                y.sum().backward()
                outs["single"] = ([torch.stack(ts) for ts in zip(*[_flat(s) for s in steps])], leaf.grad.clone())
            except (NotImplementedError, ValueError, AssertionError, IndexError, RuntimeError):   # a sequence-only neuron: both arms must refuse
                outs["single"] = "refused"
        F_.reset_net(m)
        F_.set_step_mode(m, "m")
        torch.manual_seed(1)
        leaf = x0.clone().requires_grad_(True)
        ym = m(leaf * 1.0)
        (_first(ym) if torch.is_tensor(_first(ym)) else torch.stack(list(ym))).sum().backward()
        outs["multi"] = (_flat(ym), leaf.grad.clone())
        F_.reset_net(m)
        results.append(outs)
    ours, ref = results
    assert ours.keys() == ref.keys()
    for mode in ours:
        if isinstance(ours[mode], str) or isinstance(ref[mode], str):
            assert isinstance(ours[mode], str) and isinstance(ref[mode], str), (name, mode, ours[mode] if isinstance(ours[mode], str) else "ran",
                                                                                 ref[mode] if isinstance(ref[mode], str) else "ran")
            continue
        (ya, ga), (yb, gb) = ours[mode], ref[mode]
        assert len(ya) == len(yb), (name, mode)
        for ta, tb in zip(ya, yb):
            assert ta.shape == tb.shape and torch.allclose(ta, tb, atol=1e-5, rtol=1e-5), (name, mode, float((ta - tb).abs().max()))
        assert torch.allclose(ga, gb, atol=1e-5, rtol=1e-4), (name, mode, "grad", float((ga - gb).abs().max()))
