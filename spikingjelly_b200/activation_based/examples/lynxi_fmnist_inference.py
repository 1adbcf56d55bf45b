"""Inference of the Fashion-MNIST convolutional SNN on a Lynxi chip (role of ``examples/lynxi_fmnist_inference.py`` in the
reference): the trained ``conv_fashion_mnist.CSNN`` is rewritten module by module into the operators the Lynxi compiler
accepts (``lynxi_exchange.to_lynxi_supported_modules``: time folded into the batch, neurons unrolled over T), checked against
the original network on the host, compiled and run on the device.  Without the vendor runtime (``lyngor`` / ``lynpy``) the
script stops after the host check.

    python -m spikingjelly_b200.activation_based.examples.lynxi_fmnist_inference --synthetic --channels 8 [--pt-path checkpoint_max.pth]
"""
import argparse

import torch
import torch.nn as nn

from .. import functional, lynxi_exchange
from . import conv_fashion_mnist
from ._common import synthetic_images


class InferenceNet(nn.Module):
    """``[N, C, H, W]`` image -> firing rates ``[N, classes]`` through modules that work on ``[T * N, ...]``."""

    def __init__(self, T: int, modules_list: list):
        super().__init__()
        self.T = T
        self.module_list = nn.Sequential(*modules_list)

    def forward(self, x: torch.Tensor):
        x = self.module_list(x.unsqueeze(0).expand(self.T, *x.shape).flatten(0, 1))      # the image repeated T times, time-major
        return x.reshape(self.T, x.shape[0] // self.T, -1).mean(0)


def main(argv=None):
    p = argparse.ArgumentParser(description=__doc__)
    p.add_argument("-T", type=int, default=4)
    p.add_argument("-b", "--batch-size", type=int, default=16)
    p.add_argument("--channels", type=int, default=128)
    p.add_argument("--data-dir", default="./data")
    p.add_argument("--synthetic", action="store_true")
    p.add_argument("--max-steps", type=int, default=0)
    p.add_argument("--pt-path", default=None, help="checkpoint of conv_fashion_mnist.CSNN ({'net': state_dict}); random weights if absent")
    p.add_argument("--out-model-path", default="./lynxi_model")
    p.add_argument("--lynxi-device", type=int, default=0)
    args = p.parse_args(argv)
    net_sj = conv_fashion_mnist.CSNN(args.T, args.channels, "torch").eval()
    if args.pt_path:
        ckp = torch.load(args.pt_path, map_location="cpu", weights_only=True)
        net_sj.load_state_dict(ckp["net"] if "net" in ckp else ckp)
    net = InferenceNet(args.T, lynxi_exchange.to_lynxi_supported_modules(net_sj.conv_fc, args.T)).eval()
    if args.synthetic:
        test_set = synthetic_images(4 * args.batch_size, (1, 28, 28), 10, seed=1)
    else:
        import torchvision
        test_set = torchvision.datasets.FashionMNIST(args.data_dir, train=False, transform=torchvision.transforms.ToTensor(), download=True)
    loader = torch.utils.data.DataLoader(test_set, batch_size=args.batch_size, shuffle=False, drop_last=True)
    # host check: the rewritten network must give the firing rates of the original one
    x0, _ = next(iter(loader))
    with torch.no_grad():
        want = net_sj(x0)
        functional.reset_net(net_sj)
        got = net(x0)
    gap = float((want - got).abs().max())
    print(f"host check: max |original - rewritten| = {gap:.3g}")
    result = {"host_max_abs_diff": gap}
    try:
        path = lynxi_exchange.compile_lynxi_model(args.out_model_path, net, in_data_type="float16", out_data_type="float16",
                                                  input_shape_dict={"x": torch.Size([args.batch_size, 1, 28, 28])})
        net_lynxi = lynxi_exchange.load_lynxi_model(args.lynxi_device, path)
    except ImportError as exc:
        print(f"device run skipped: {exc}")
        result["device"] = None
        return result
    seen = correct = 0
    with torch.no_grad():
        for step, (img, label) in enumerate(loader):
            if args.max_steps and step >= args.max_steps:
                break
            y = net_lynxi(lynxi_exchange.torch_tensor_to_lynxi(img.half(), args.lynxi_device))
            y = lynxi_exchange.lynxi_tensor_to_torch(y, shape=[label.shape[0], 10], dtype="float16")
            correct += (y.argmax(1) == label).sum().item()
            seen += img.shape[0]
    result["device"] = {"accuracy": correct / max(seen, 1)}
    print(f"lynxi inference accuracy = {result['device']['accuracy']}")
    return result


if __name__ == "__main__":
    main()
