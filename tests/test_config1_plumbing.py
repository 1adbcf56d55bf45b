"""Single-layer SNN plumbing run on CPU: Flatten -> Linear(784, 10) -> LIF, T=4, Poisson
input, MSE on the firing rate, SGD lr 0.1 for 10 steps.  Our eager path must reproduce the
reference's eager path bit for bit (same seed, same op order)."""
import torch
import torch.nn as nn
import torch.nn.functional as F

from spikingjelly_b200.activation_based import encoding, functional, layer, neuron, surrogate


def _run(ns, steps=10, T=4, B=64):
    torch.manual_seed(0)
    net = nn.Sequential(ns.layer.Flatten(), ns.layer.Linear(784, 10, bias=False),
                        ns.neuron.LIFNode(tau=2.0, v_threshold=1.0, v_reset=0.0,
                                          surrogate_function=ns.surrogate.ATan(alpha=2.0)))
    ns.functional.set_step_mode(net, "m")
    enc = ns.encoding.PoissonEncoder()
    opt = torch.optim.SGD(net.parameters(), lr=0.1)
    losses = []
    for _ in range(steps):
        img = torch.rand(B, 1, 28, 28)
        label = torch.randint(0, 10, (B,))
        x_seq = torch.stack([enc(img) for _ in range(T)])
        rate = net(x_seq).mean(0)
        loss = F.mse_loss(rate, F.one_hot(label, 10).float())
        opt.zero_grad()
        loss.backward()
        opt.step()
        ns.functional.reset_net(net)
        losses.append(loss.item())
    return losses, net[1].weight.detach().clone()


class _Ours:
    neuron, layer, functional, surrogate, encoding = neuron, layer, functional, surrogate, encoding


def test_config1_runs_and_learns():
    losses, w = _run(_Ours)
    assert all(torch.isfinite(torch.tensor(losses)))
    assert losses[-1] <= losses[0]


def test_config1_bit_exact_vs_reference(reference):
    ours_l, ours_w = _run(_Ours)
    ref_l, ref_w = _run(reference)
    assert ours_l == ref_l
    assert torch.equal(ours_w, ref_w)
