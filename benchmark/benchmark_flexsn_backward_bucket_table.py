#!/usr/bin/env python
"""Which tensor sizes the generated FlexSN kernels meet in spiking VGG networks, grouped into size buckets, and the time and
memory rate of the generated forward and backward kernel for every distinct size.  Counterpart of the reference's
``benchmark/benchmark_flexsn_backward_bucket_table.py`` (there the buckets select Triton launch configurations; the CUDA
generator has one configuration, so the table shows how its memory rate changes with the size).

    python benchmark/benchmark_flexsn_backward_bucket_table.py [--workloads cifar_vgg11_bn imagenet_vgg11_bn imagenet_vgg16_bn]
"""
import argparse
import json
import sys
from collections import Counter
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(Path(__file__).resolve().parent))
import _arms  # noqa: E402

BUCKETS = ((4096, "small (<= 4096)"), (131072, "medium (4097..131072)"), (1048576, "large (131073..1048576)"),
           (8388608, "xlarge (1048577..8388608)"), (float("inf"), "xxlarge (> 8388608)"))


def bucket_of(n: int) -> str:
    return next(label for top, label in BUCKETS if n <= top)


def main():
    from spikingjelly_b200.activation_based import functional, neuron, surrogate
    from spikingjelly_b200.activation_based.model import spiking_vgg
    from spikingjelly_b200.ops import flexsn as K
    ap = argparse.ArgumentParser()
    ap.add_argument("--workloads", nargs="+", default=["cifar_vgg11_bn", "imagenet_vgg11_bn", "imagenet_vgg16_bn"])
    ap.add_argument("--iters", type=int, default=20)
    a = ap.parse_args()
    sg = surrogate.Sigmoid(alpha=4.0)

    def core(x, v):
        h = v + (x - v) / 2.0
        s = sg(h - 1.0)
        return s, h * (1.0 - s)

    def flexsn(**kw):
        return neuron.FlexSN(core=core, num_inputs=1, num_states=1, num_outputs=1, step_mode=kw.get("step_mode", "m"), backend="cuda")
    table = {"cifar_vgg11_bn": (spiking_vgg.spiking_vgg11_bn, 10, (4, 32, 3, 32, 32)),
             "imagenet_vgg11_bn": (spiking_vgg.spiking_vgg11_bn, 1000, (4, 8, 3, 224, 224)),
             "imagenet_vgg16_bn": (spiking_vgg.spiking_vgg16_bn, 1000, (4, 8, 3, 224, 224))}
    sizes, kernel = Counter(), None
    for name in a.workloads:
        build, classes, shape = table[name]
        net = build(spiking_neuron=flexsn, num_classes=classes, step_mode="m").cuda().eval()
        functional.set_step_mode(net, "m")
        seen = []
        hooks = [m.register_forward_pre_hook(lambda mod, inp, seen=seen: seen.append((inp[0].shape[0], inp[0][0].numel())))
                 for m in net.modules() if isinstance(m, neuron.FlexSN)]
        with torch.no_grad():
            net(torch.randn(shape, device="cuda"))
        for h in hooks:
            h.remove()
        kernel = kernel or next(K.lookup_kernel_handle(m._handle) for m in net.modules() if isinstance(m, neuron.FlexSN))
        per_bucket = Counter(bucket_of(n) for _, n in seen)
        print(json.dumps({"workload": name, "flexsn_layers": len(seen), "layers_per_bucket": dict(per_bucket)}), flush=True)
        sizes.update(seen)
        functional.reset_net(net)
        del net
        torch.cuda.empty_cache()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for (T, n), count in sorted(sizes.items(), key=lambda kv: kv[0][1]):
        x, g, s0 = torch.randn(T, n, device="cuda"), torch.randn(T, n, device="cuda"), torch.zeros(n, device="cuda")
        _, seqs, _ = kernel.forward([x], [s0], True)
        f = _arms.summary(_arms.time_cuda(lambda: kernel.forward([x], [s0], True), 3, a.iters, flush=flush))["median_ms"] * 1e3
        b = _arms.summary(_arms.time_cuda(lambda: kernel.backward([x], [s0], seqs, [g], [None], [None], [True, False]), 3, a.iters, flush=flush))["median_ms"] * 1e3
        byte = T * n * 4
        print(json.dumps({"T": T, "neurons": n, "bucket": bucket_of(n), "layers": count, "forward_us": round(f, 1), "backward_us": round(b, 1),
                          "forward_gb_s": round(3 * byte / f / 1e3, 1), "backward_gb_s": round(4 * byte / b / 1e3, 1)}), flush=True)


if __name__ == "__main__":
    main()
