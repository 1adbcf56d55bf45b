"""DVS128 Gesture classification with the PLIF network of the model zoo: events are integrated to T frames by the dataset
class, the network runs in multi-step mode (role of ``examples/classify_dvsg.py`` in the reference).

    python -m spikingjelly_b200.activation_based.examples.classify_dvsg --synthetic --max-steps 10 -T 8 --channels 32
"""
import argparse

import torch
import torch.nn.functional as F
from torch.utils.data import TensorDataset

from .. import functional, neuron, surrogate
from ...models import parametric_lif_net
from ._common import add_common_args, loaders, pick_backend, pick_device, run_epochs


def main(argv=None):
    p = add_common_args(argparse.ArgumentParser(description=__doc__))
    p.add_argument("-T", type=int, default=16)
    p.add_argument("--channels", type=int, default=128)
    args = p.parse_args(argv)
    device = pick_device(args.device)
    if args.synthetic:
        g = torch.Generator().manual_seed(0)
        def fake(n, seed):
            y = torch.randint(0, 11, (n,), generator=g)
            x = (torch.rand(n, args.T, 2, 128, 128, generator=g) < (0.02 + 0.01 * y.view(-1, 1, 1, 1, 1))).float()
            return TensorDataset(x, y)
        train_set, test_set = fake(64, 0), fake(32, 1)
    else:
        from ...datasets.dvs128_gesture import DVS128Gesture
        kw = dict(data_type="frame", frames_number=args.T, split_by="number")
        train_set, test_set = DVS128Gesture(args.data_dir, train=True, **kw), DVS128Gesture(args.data_dir, train=False, **kw)
    net = parametric_lif_net.DVSGestureNet(channels=args.channels, spiking_neuron=neuron.LIFNode, surrogate_function=surrogate.ATan(),
                                           detach_reset=True)
    functional.set_step_mode(net, "m")
    functional.set_backend(net, pick_backend(device, args.backend), instance=neuron.LIFNode)
    net.to(device)
    forward = lambda n, x: n(x.transpose(0, 1)).mean(0)           # [N, T, ...] -> [T, N, ...]
    loss_fn = lambda out, y: F.mse_loss(out, F.one_hot(y, 11).float())
    return run_epochs(net, *loaders(train_set, test_set, args), forward, loss_fn, args, device)


if __name__ == "__main__":
    main()
