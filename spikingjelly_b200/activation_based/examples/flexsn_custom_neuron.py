"""A neuron that does not exist in the library — adaptive-threshold LIF with two states — written as a plain PyTorch step
function and compiled by FlexSN into one CUDA kernel per direction (role of ``model/train_flexsn_inductor_example.py``).

    python -m spikingjelly_b200.activation_based.examples.flexsn_custom_neuron
"""
import argparse
import time

import torch

from .. import surrogate
from ..neuron.flexsn import FlexSN

_sg = surrogate.ATan()


def adaptive_lif(x, v, a):
    """v: membrane potential, a: threshold adaptation that jumps on every spike and decays otherwise."""
    h = v + (x - v) / 2.0
    s = _sg(h - (1.0 + a))
    return s, h * (1.0 - s), a * 0.9 + s * 0.2


def main(argv=None):
    p = argparse.ArgumentParser(description=__doc__)
    p.add_argument("-T", type=int, default=8)
    p.add_argument("-N", type=int, default=1 << 20)
    args = p.parse_args(argv)
    device = "cuda" if torch.cuda.is_available() else "cpu"
    x = torch.rand(args.T, args.N, device=device) * 2
    compiled = FlexSN(adaptive_lif, num_inputs=1, num_states=2, num_outputs=1, backend="triton")
    eager = FlexSN(adaptive_lif, num_inputs=1, num_states=2, num_outputs=1, backend="torch")
    print("kernel available:", compiled.kernel_available, "| device:", device)
    for name, m in (("compiled", compiled), ("eager", eager)):
        xi = x.clone().requires_grad_(True)
        t0 = time.time()
        s = m(xi)
        s.sum().backward()
        if device == "cuda":
            torch.cuda.synchronize()
        print(f"{name}: firing rate {s.mean().item():.4f}, grad norm {xi.grad.norm().item():.4f}, {1e3 * (time.time() - t0):.1f} ms")
        m.reset()


if __name__ == "__main__":
    main()
