"""ANN -> SNN conversion of a CIFAR-10 ResNet-18 (3x3 stem, residual additions kept as graph nodes) with the rate-coding recipe
in ``Max`` mode: accuracy of the source network and of the converted network over T steps.  Role of
``spikingjelly/activation_based/ann2snn/examples/resnet18_cifar10.py``.

    python -m spikingjelly_b200.activation_based.ann2snn.examples.resnet18_cifar10 --synthetic --time-steps 16
"""
import argparse
import os

import torch
import torch.nn as nn

from ... import ann2snn
from ._common import add_common_args, ann_accuracy, class_blobs, curve_summary, fit, loaders, report, snn_accuracy_curve


class BasicBlock(nn.Module):
    def __init__(self, cin, cout, stride):
        super().__init__()
        self.conv1, self.bn1, self.relu1 = nn.Conv2d(cin, cout, 3, stride, 1, bias=False), nn.BatchNorm2d(cout), nn.ReLU()
        self.conv2, self.bn2, self.relu2 = nn.Conv2d(cout, cout, 3, 1, 1, bias=False), nn.BatchNorm2d(cout), nn.ReLU()
        self.shortcut = nn.Sequential() if stride == 1 and cin == cout else nn.Sequential(nn.Conv2d(cin, cout, 1, stride, bias=False), nn.BatchNorm2d(cout))

    def forward(self, x):
        return self.relu2(self.bn2(self.conv2(self.relu1(self.bn1(self.conv1(x))))) + self.shortcut(x))


class ResNet18(nn.Module):
    def __init__(self, width: int = 64, classes: int = 10):
        super().__init__()
        self.stem = nn.Sequential(nn.Conv2d(3, width, 3, 1, 1, bias=False), nn.BatchNorm2d(width), nn.ReLU())
        blocks, cin = [], width
        for i, stride in enumerate((1, 2, 2, 2)):
            cout = width * 2 ** i
            blocks += [BasicBlock(cin, cout, stride), BasicBlock(cout, cout, 1)]
            cin = cout
        self.layers = nn.Sequential(*blocks)
        self.pool, self.flatten, self.fc = nn.AdaptiveAvgPool2d(1), nn.Flatten(), nn.Linear(cin, classes)

    def forward(self, x):
        return self.fc(self.flatten(self.pool(self.layers(self.stem(x)))))


def main(argv=None):
    p = add_common_args(argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter))
    p.add_argument("--dataset-dir", default="./data/cifar10")
    p.add_argument("--checkpoint-path", default="./SJ-cifar10-resnet18_model-sample.pth")
    p.add_argument("--batch-size", type=int, default=100)
    p.add_argument("--time-steps", type=int, default=400)
    p.add_argument("--max-eval-batches", type=int, default=None)
    args = p.parse_args(argv)
    torch.manual_seed(args.seed)
    device = torch.device(args.device)
    if args.synthetic:
        train_set, test_set = class_blobs(600, (3, 32, 32), 10, seed=1), class_blobs(200, (3, 32, 32), 10, seed=2)
    else:
        import torchvision
        tf = torchvision.transforms.Compose([torchvision.transforms.ToTensor(), torchvision.transforms.Normalize((0.4914, 0.4822, 0.4465), (0.2023, 0.1994, 0.2010))])
        train_set = torchvision.datasets.CIFAR10(args.dataset_dir, train=True, transform=tf, download=True)
        test_set = torchvision.datasets.CIFAR10(args.dataset_dir, train=False, transform=tf, download=True)
    train_loader, test_loader = loaders(train_set, test_set, args.batch_size)
    ann = ResNet18(16 if args.synthetic else 64).to(device)
    if not args.synthetic and os.path.exists(args.checkpoint_path):
        ann.load_state_dict(torch.load(args.checkpoint_path, map_location=device, weights_only=True))
    else:
        fit(ann, train_loader, device, epochs=3 if args.synthetic else 1, lr=1e-2 if args.synthetic else 1e-3)
    ann.eval()
    snn = ann2snn.Converter(recipe=ann2snn.RateCodingRecipe(dataloader=train_loader, mode="Max"), device=device).convert(ann)
    curve = snn_accuracy_curve(snn, test_loader, device, args.time_steps, args.max_eval_batches)
    return report({"time_steps": args.time_steps, "ann_accuracy": round(ann_accuracy(ann, test_loader, device, args.max_eval_batches), 4),
                   "snn_accuracy": round(curve[-1], 4), "curve": curve_summary(curve, (1, 2, 4, 8, 16, 32, 64, 128, 256, 400))}, args.output)


if __name__ == "__main__":
    main()
