"""Trace-based STDP on one synapse: a presynaptic and a postsynaptic Poisson train drive ``STDPLearner`` and the weight
change is compared with the closed form ``trace_pre * post - trace_post * pre`` (the reference's
``examples/stdp_trace.py`` plots the same quantities).

    python -m spikingjelly_b200.activation_based.examples.stdp_trace -T 200 [--plot stdp.png]
"""
from __future__ import annotations

import argparse

import torch
import torch.nn as nn

from .. import functional, learning, neuron


def main(argv=None) -> dict:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("-T", type=int, default=200)
    p.add_argument("--tau-pre", type=float, default=20.0)
    p.add_argument("--tau-post", type=float, default=20.0)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--plot", default="", help="write the traces and the weight to this image (needs matplotlib)")
    a = p.parse_args(argv)
    torch.manual_seed(a.seed)

    fc = nn.Linear(1, 1, bias=False)
    nn.init.constant_(fc.weight, 0.4)
    sn = neuron.IFNode()
    net = nn.Sequential(fc, sn)
    learner = learning.STDPLearner("s", fc, sn, a.tau_pre, a.tau_post, f_pre=lambda w: torch.clamp(w, -1, 1.0),
                                   f_post=lambda w: torch.clamp(w, -1, 1.0))
    opt = torch.optim.SGD(net.parameters(), lr=0.01, momentum=0.0)

    pre = (torch.rand(a.T, 1, 1) < 0.2).float()
    rec = {"pre": [], "post": [], "trace_pre": [], "trace_post": [], "w": []}
    tp = tq = 0.0
    expect_w = float(fc.weight.detach())
    with torch.no_grad():
        for t in range(a.T):
            opt.zero_grad()
            w_now = float(fc.weight)
            post = net(pre[t])
            learner.step(on_grad=True)
            # the same update by hand: traces decay, then take this step's spikes
            tp = tp - tp / a.tau_pre + float(pre[t])
            tq = tq - tq / a.tau_post + float(post)
            dw = tp * float(post) * max(min(w_now, 1.0), -1.0) - tq * float(pre[t]) * max(min(w_now, 1.0), -1.0)
            expect_w = expect_w + 0.01 * dw                 # the learner writes -delta_w into grad; SGD subtracts it
            opt.step()
            rec["pre"].append(float(pre[t])); rec["post"].append(float(post))
            rec["trace_pre"].append(float(learner.trace_pre)); rec["trace_post"].append(float(learner.trace_post))
            rec["w"].append(float(fc.weight))
    functional.reset_net(net)
    learner.reset()
    err = abs(rec["w"][-1] - expect_w)
    print(f"T {a.T}: {int(sum(rec['pre']))} pre spikes, {int(sum(rec['post']))} post spikes, w 0.4 -> {rec['w'][-1]:.5f} "
          f"(closed form {expect_w:.5f}, |diff| {err:.2e})")
    if a.plot:
        from ...visualizing import _utils
        plt = _utils.pyplot()
        fig, ax = plt.subplots(5, 1, figsize=(8, 8), sharex=True)
        for i, k in enumerate(("pre", "trace_pre", "post", "trace_post", "w")):
            ax[i].plot(rec[k]) if "trace" in k or k == "w" else ax[i].eventplot([t for t, s in enumerate(rec[k]) if s])
            ax[i].set_ylabel(k)
        fig.savefig(a.plot, dpi=150)
    return {"w_final": rec["w"][-1], "w_expected": expect_w, "post_spikes": sum(rec["post"])}


if __name__ == "__main__":
    main()
