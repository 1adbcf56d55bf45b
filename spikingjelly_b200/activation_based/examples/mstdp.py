"""Reward-modulated STDP (``MSTDPLearner`` / ``MSTDPETLearner``) on a one-layer network: the reward is +1 when the
target output neuron fired more than the others in the last window and -1 otherwise, so the weights toward the target
grow (the reference's ``examples/mstdp.py`` and ``examples/mstdpet.py`` run the two learners on a fixed reward trace).

    python -m spikingjelly_b200.activation_based.examples.mstdp [--eligibility-trace] -T 200
"""
from __future__ import annotations

import argparse

import torch
import torch.nn as nn

from .. import functional, learning, neuron


def main(argv=None) -> dict:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("-T", type=int, default=200)
    p.add_argument("-N", "--batch", type=int, default=4)
    p.add_argument("--n-in", type=int, default=16)
    p.add_argument("--n-out", type=int, default=4)
    p.add_argument("--target", type=int, default=1)
    p.add_argument("--eligibility-trace", action="store_true", help="MSTDPET (reward times a low-passed eligibility) instead of MSTDP")
    p.add_argument("--tau-trace", type=float, default=10.0)
    p.add_argument("--lr", type=float, default=0.05)
    p.add_argument("--seed", type=int, default=0)
    a = p.parse_args(argv)
    torch.manual_seed(a.seed)

    fc = nn.Linear(a.n_in, a.n_out, bias=False)
    nn.init.uniform_(fc.weight, 0.2, 0.4)
    sn = neuron.LIFNode(tau=2.0)
    net = nn.Sequential(fc, sn)
    clamp = lambda w: torch.clamp(w, 0.0, 1.0)          # noqa: E731
    if a.eligibility_trace:
        learner = learning.MSTDPETLearner("s", fc, sn, 5.0, 5.0, a.tau_trace, f_pre=clamp, f_post=clamp)
    else:
        learner = learning.MSTDPLearner("s", a.batch, fc, sn, 5.0, 5.0, f_pre=clamp, f_post=clamp)
    opt = torch.optim.SGD(net.parameters(), lr=a.lr)
    w0 = fc.weight.detach().clone()

    # the eligibility-trace learner works on one sample at a time (unbatched spikes, scalar reward)
    lead = () if a.eligibility_trace else (a.batch,)
    counts = torch.zeros(*lead, a.n_out)
    with torch.no_grad():
        for t in range(a.T):
            x = (torch.rand(*lead, a.n_in) < 0.3).float()
            out = net(x)
            counts = 0.9 * counts + out
            others = torch.cat([counts[..., :a.target], counts[..., a.target + 1:]], -1).max(-1).values
            reward = torch.where(counts[..., a.target] >= others, 1.0, -1.0)
            opt.zero_grad()
            learner.step(float(reward) if a.eligibility_trace else reward, on_grad=True)
            if fc.weight.grad is not None:
                # only the target neuron's own synapses are trained here: mask the other rows of the update
                mask = torch.zeros_like(fc.weight)
                mask[a.target] = 1.0
                fc.weight.grad.mul_(mask)
                opt.step()
                fc.weight.clamp_(0.0, 1.0)
    functional.reset_net(net)
    learner.reset()
    dw = (fc.weight.detach() - w0)
    print(f"{'MSTDPET' if a.eligibility_trace else 'MSTDP'}: mean weight change of the target row {dw[a.target].mean():+.4f}, "
          f"others {dw[[i for i in range(a.n_out) if i != a.target]].abs().max():.4f}")
    return {"target_dw": float(dw[a.target].mean()), "other_dw": float(dw.abs().sum() - dw[a.target].abs().sum())}


if __name__ == "__main__":
    main()
