"""MNIST classifier made of ``lava_exchange.BlockContainer`` blocks (a synapse without bias + an IF neuron, trained with 8-bit
quantised weights), Poisson-encoded input, then exported to lava-dl slayer blocks and to the HDF5 network file Lava loads
(role of ``examples/lava_mnist.py`` in the reference).  Training and evaluation need nothing beyond this package; the
export needs ``lava-dl`` and ``h5py`` and is skipped with a message where they are absent.

    python -m spikingjelly_b200.activation_based.examples.lava_mnist --synthetic --max-steps 20 -T 8
"""
import argparse
import os

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import encoding, functional, lava_exchange, neuron, surrogate
from ._common import add_common_args, loaders, pick_device, run_epochs, synthetic_images


def export_hdf5(net, filename):
    """Every slayer block writes its own group ``layer/<i>``."""
    import h5py
    with h5py.File(filename, "w") as h:
        group = h.create_group("layer")
        for i, block in enumerate(net):
            block.export_hdf5(group.create_group(f"{i}"))


class MNISTNet(nn.Module):
    def __init__(self, channels: int = 16):
        super().__init__()
        sn = lambda: neuron.IFNode(surrogate_function=surrogate.ATan(), detach_reset=True)      # noqa: E731
        conv = lambda i, o, k, s, p: lava_exchange.BlockContainer(nn.Conv2d(i, o, k, s, p, bias=False), sn())   # noqa: E731
        self.conv_fc = nn.Sequential(
            conv(1, channels, 3, 1, 1), conv(channels, channels, 2, 2, 0),            # 28 -> 14
            conv(channels, channels, 3, 1, 1), conv(channels, channels, 2, 2, 0),     # 14 -> 7
            lava_exchange.BlockContainer(nn.Flatten(), None),
            lava_exchange.BlockContainer(nn.Linear(channels * 7 * 7, 128, bias=False), sn()),
            lava_exchange.BlockContainer(nn.Linear(128, 10, bias=False), sn()))

    def to_lava(self):
        return nn.Sequential(*[m.to_lava_block() for m in self.conv_fc if isinstance(m, lava_exchange.BlockContainer)])

    def forward(self, x):
        return self.conv_fc(x)


def main(argv=None):
    p = add_common_args(argparse.ArgumentParser(description=__doc__))
    p.add_argument("-T", type=int, default=16)
    p.add_argument("--channels", type=int, default=16)
    p.add_argument("--out-dir", default="./")
    p.set_defaults(lr=1e-3)
    args = p.parse_args(argv)
    device = pick_device(args.device)
    if args.synthetic:
        train_set, test_set = synthetic_images(1024, (1, 28, 28), 10), synthetic_images(256, (1, 28, 28), 10, seed=1)
    else:
        import torchvision
        tf = torchvision.transforms.ToTensor()
        train_set = torchvision.datasets.MNIST(args.data_dir, train=True, transform=tf, download=True)
        test_set = torchvision.datasets.MNIST(args.data_dir, train=False, transform=tf, download=True)
    net = MNISTNet(args.channels).to(device)
    functional.set_step_mode(net, "m")
    encoder = encoding.PoissonEncoder(step_mode="m")
    train, test = loaders(train_set, test_set, args)
    rate = lambda n, x: n(encoder(x.unsqueeze(0).expand(args.T, *x.shape))).mean(0)       # noqa: E731
    stats = run_epochs(net, train, test, rate, F.cross_entropy, args, device)
    print("test acc[sj] =", stats.get("test_acc"))
    os.makedirs(args.out_dir, exist_ok=True)
    torch.save(net.state_dict(), os.path.join(args.out_dir, "net.pt"))
    try:
        net_ladl = net.to_lava().to(device).eval()
    except ImportError as exc:
        print(f"export skipped: {exc}")
        stats["exported"] = False
        return stats
    seen = correct = 0
    with torch.no_grad():
        for step, (x, y) in enumerate(test):
            if args.max_steps and step >= args.max_steps:
                break
            x, y = x.to(device), y.to(device)
            spikes = lava_exchange.TNX_to_NXT(encoder(x.unsqueeze(0).expand(args.T, *x.shape)))
            correct += (net_ladl(spikes).mean(-1).argmax(1) == y).sum().item()
            seen += y.numel()
    stats["lava_test_acc"] = correct / max(seen, 1)
    print("test acc[lava dl] =", stats["lava_test_acc"])
    torch.save(net_ladl.state_dict(), os.path.join(args.out_dir, "net_ladl.pt"))
    export_hdf5(net_ladl, os.path.join(args.out_dir, "net_la.net"))
    stats["exported"] = True
    return stats


if __name__ == "__main__":
    main()
