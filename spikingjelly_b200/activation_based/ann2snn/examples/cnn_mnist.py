"""ANN -> SNN conversion of a small MNIST CNN: the rate-coding recipe in its threshold modes (``max``, ``99.9%`` robust
percentile, ``1/2`` ... ``1/5`` scaled maximum) next to local threshold balancing, each reported as accuracy of the source
network, accuracy of the converted network after T steps and the accuracy-over-time curve.  Role of
``spikingjelly/activation_based/ann2snn/examples/cnn_mnist.py``.

    python -m spikingjelly_b200.activation_based.ann2snn.examples.cnn_mnist --synthetic --time-steps 32
    python -m spikingjelly_b200.activation_based.ann2snn.examples.cnn_mnist --dataset-dir ./data/mnist [--checkpoint-path ann.pth]
"""
import argparse
import os

import torch
import torch.nn as nn

from ... import ann2snn
from ._common import add_common_args, ann_accuracy, class_blobs, curve_summary, fit, loaders, report, snn_accuracy_curve


class ANN(nn.Module):
    """Three convolution blocks (conv - batch norm - ReLU - average pooling) and a linear classifier."""

    def __init__(self, channels: int = 32):
        super().__init__()
        c = channels
        self.network = nn.Sequential(
            nn.Conv2d(1, c, 3, 1), nn.BatchNorm2d(c), nn.ReLU(), nn.AvgPool2d(2, 2),
            nn.Conv2d(c, c, 3, 1), nn.BatchNorm2d(c), nn.ReLU(), nn.AvgPool2d(2, 2),
            nn.Conv2d(c, c, 3, 1), nn.BatchNorm2d(c), nn.ReLU(), nn.AvgPool2d(2, 2),
            nn.Flatten(), nn.Linear(c, 10))

    def forward(self, x):
        return self.network(x)


def parse_args(argv=None):
    p = add_common_args(argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter))
    p.add_argument("--dataset-dir", default="./data/mnist")
    p.add_argument("--batch-size", type=int, default=100)
    p.add_argument("--test-batch-size", type=int, default=50)
    p.add_argument("--time-steps", type=int, default=32)
    p.add_argument("--epochs", type=int, default=1, help="training epochs of the source network when no checkpoint is given")
    p.add_argument("--checkpoint-path", default=None, help="state dict of a trained ANN (written after training when absent)")
    p.add_argument("--max-eval-batches", type=int, default=None)
    p.add_argument("--skip-mode-sweep", action="store_true")
    return p.parse_args(argv)


def convert_and_eval(recipe, device, ann, test_loader, time_steps, max_batches=None):
    snn = ann2snn.Converter(recipe=recipe, device=device).convert(ann)
    curve = snn_accuracy_curve(snn, test_loader, device, time_steps, max_batches)
    return {"snn_accuracy": round(curve[-1], 4), "curve": curve_summary(curve)}


def main(argv=None):
    args = parse_args(argv)
    torch.manual_seed(args.seed)
    device = torch.device(args.device)
    if args.synthetic:
        train_set, test_set = class_blobs(2000, (1, 28, 28), 10, seed=1), class_blobs(500, (1, 28, 28), 10, seed=2)
    else:
        import torchvision
        tf = torchvision.transforms.ToTensor()
        train_set = torchvision.datasets.MNIST(args.dataset_dir, train=True, transform=tf, download=True)
        test_set = torchvision.datasets.MNIST(args.dataset_dir, train=False, transform=tf, download=True)
    train_loader, test_loader = loaders(train_set, test_set, args.batch_size, args.test_batch_size)
    ann = ANN(16 if args.synthetic else 32).to(device)
    if args.checkpoint_path and os.path.exists(args.checkpoint_path):
        ann.load_state_dict(torch.load(args.checkpoint_path, map_location=device, weights_only=True))
    else:
        fit(ann, train_loader, device, epochs=4 if args.synthetic else args.epochs, lr=1e-2 if args.synthetic else 1e-3)
        if args.checkpoint_path:
            torch.save(ann.state_dict(), args.checkpoint_path)
    ann.eval()
    results = {"time_steps": args.time_steps, "ann_accuracy": round(ann_accuracy(ann, test_loader, device, args.max_eval_batches), 4)}
    recipes = {
        "rate_max": lambda: ann2snn.RateCodingRecipe(dataloader=train_loader, mode="max"),
        "rate_99.9%": lambda: ann2snn.RateCodingRecipe(dataloader=train_loader, mode="99.9%"),
        "local_threshold_balancing": lambda: ann2snn.LocalThresholdBalancingRecipe(dataloader=train_loader),
    }
    if not args.skip_mode_sweep:
        recipes.update({f"rate_1/{k}": (lambda k=k: ann2snn.RateCodingRecipe(dataloader=train_loader, mode=1.0 / k)) for k in (2, 3, 4, 5)})
    results["recipes"] = {name: convert_and_eval(make(), device, ann, test_loader, args.time_steps, args.max_eval_batches) for name, make in recipes.items()}
    return report(results, args.output)


if __name__ == "__main__":
    main()
