#!/usr/bin/env python
"""Spiking VGG-16-BN (CIFAR-sized input, T 4, batch 64) with three neurons: ``LIFNode`` on the eager backend, ``LIFNode`` on the
kernel backend, and a ``FlexSN`` whose LIF step function is compiled by the generator; one full training step
(``--mode train``: forward, cross-entropy, backward, SGD) or a gradient-free forward (``--mode inference``).  Counterpart of the
reference's ``benchmark/flexsn/benchmark_vgg_train.py`` and ``benchmark_vgg_inductor.py``.

    python benchmark/benchmark_flexsn_vgg.py [--mode train|inference] [--impl ours|reference] [--T 4 --batch 64]
"""
import argparse
import gc
import json
import sys
from pathlib import Path

import torch
import torch.nn as nn

sys.path.insert(0, str(Path(__file__).resolve().parent))
import _arms  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--mode", choices=["train", "inference"], default="train")
    ap.add_argument("--T", type=int, default=4)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--image", type=int, default=32)
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    a = ap.parse_args()
    try:
        arm = _arms.load(a.impl)
        neuron, functional, surrogate = arm.get("neuron"), arm.get("functional"), arm.get("surrogate")
        vgg = arm.get("model.spiking_vgg").spiking_vgg16_bn
    except Exception as exc:
        return _arms.unavailable(a.impl, exc)
    sg = surrogate.Sigmoid(alpha=4.0)

    def lif_core(x, v):
        h = v + (x - v) / 2.0
        s = sg(h - 1.0)
        return s, h * (1.0 - s)
    generated = "cuda" if a.impl == "ours" else "inductor"

    def flexsn(**kw):
        return neuron.FlexSN(core=lif_core, num_inputs=1, num_states=1, num_outputs=1, step_mode=kw.get("step_mode", "m"), backend=generated)
    configs = [("LIFNode backend=torch", lambda: vgg(spiking_neuron=neuron.LIFNode, step_mode="m", backend="torch", surrogate_function=sg)),
               (f"LIFNode backend={arm.fast_backend}", lambda: vgg(spiking_neuron=neuron.LIFNode, step_mode="m", backend=arm.fast_backend, surrogate_function=sg)),
               (f"FlexSN backend={generated}", lambda: vgg(spiking_neuron=flexsn, step_mode="m"))]
    torch.manual_seed(0)
    x = torch.randn(a.T, a.batch, 3, a.image, a.image, device="cuda")
    y = torch.randint(0, 1000, (a.batch,), device="cuda")
    rows, base = [], None
    for label, build in configs:
        try:
            net = build().cuda()
            functional.set_step_mode(net, "m")
            opt = torch.optim.SGD(net.parameters(), lr=0.01)

            def step():
                functional.reset_net(net)
                if a.mode == "inference":
                    with torch.no_grad():
                        return net(x)
                opt.zero_grad(set_to_none=True)
                out = net(x)
                out = out.mean(0) if out.dim() == 3 else out
                nn.functional.cross_entropy(out, y).backward()
                opt.step()
            net.train(a.mode == "train")
            ms = _arms.summary(_arms.time_cuda(step, a.warmup, a.iters))["median_ms"]
            base = base or ms
            rows.append({"impl": a.impl, "mode": a.mode, "neuron": label, "ms_per_iter": round(ms, 3), "images_per_s": round(a.batch / ms * 1e3, 1),
                         "vs_torch_backend": round(base / ms, 2)})
            del net, opt
        except Exception as exc:
            rows.append({"impl": a.impl, "mode": a.mode, "neuron": label, "error": f"{type(exc).__name__}: {exc}"[:200]})
        print(json.dumps(rows[-1]), flush=True)
        gc.collect()
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
