"""torchvision ResNet-18 on ImageNet converted three ways (rate coding with the maximum, with the 99.9 % percentile, local
threshold balancing with channel-wise thresholds, spiking max pooling and half-threshold initial potential), top-1 / top-5 of
each against the source network for several simulation lengths, with an optional read-out delay: steps before
``--delay-start`` run but are not accumulated (``auto`` = number of spiking layers).  Role of
``spikingjelly/activation_based/ann2snn/examples/imagenet_resnet18_ltb.py``.

    python -m spikingjelly_b200.activation_based.ann2snn.examples.imagenet_resnet18_ltb --synthetic --time-steps 8 16 --output out.json
    python -m ...imagenet_resnet18_ltb --data-root /data/imagenet --weights IMAGENET1K_V1 --output out.json
"""
import argparse

import torch
import torch.nn as nn
from torch.utils.data import DataLoader, Subset

from ... import ann2snn, functional, neuron
from ._common import add_common_args, class_blobs, report


def topk(output, target, ks=(1, 5)):
    ranked = output.topk(max(ks), dim=1).indices.cpu()
    return [float((ranked[:, :k] == target[:, None]).any(1).sum()) for k in ks]


@torch.no_grad()
def evaluate_ann(model, loader, device):
    model.eval()
    hit, total = [0.0, 0.0], 0
    for img, label in loader:
        hit = [h + c for h, c in zip(hit, topk(model(img.to(device)), label))]
        total += label.numel()
    return {"top1": hit[0] / total, "top5": hit[1] / total}


@torch.no_grad()
def evaluate_snn(model, loader, device, time_steps, delay_start=0):
    model.eval()
    hit, total = [0.0, 0.0], 0
    for img, label in loader:
        functional.reset_net(model)
        img, acc = img.to(device), 0.0
        for t in range(delay_start + time_steps):
            out = model(img)
            if t >= delay_start:
                acc = acc + out
        hit = [h + c for h, c in zip(hit, topk(acc, label))]
        total += label.numel()
    functional.reset_net(model)
    return {"top1": hit[0] / total, "top5": hit[1] / total}


def main(argv=None):
    p = add_common_args(argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter))
    p.add_argument("--data-root", default=None, help="ImageNet root with train/ and val/ folders")
    p.add_argument("--weights", default=None, help="torchvision weight name, e.g. IMAGENET1K_V1 (random weights when absent)")
    p.add_argument("--calib-samples", type=int, default=50000)
    p.add_argument("--eval-samples", type=int, default=None)
    p.add_argument("--batch-size", type=int, default=128)
    p.add_argument("--num-workers", type=int, default=8)
    p.add_argument("--time-steps", type=int, nargs="+", default=[32, 64])
    p.add_argument("--delay-start", default="0", help="an integer or 'auto'")
    p.add_argument("--recipes", nargs="+", default=["rate_max", "rate_99.9%", "ltb"], choices=["rate_max", "rate_99.9%", "ltb"])
    args = p.parse_args(argv)
    torch.manual_seed(args.seed)
    device = torch.device(args.device)
    import torchvision
    if args.synthetic:
        calib, val, classes = class_blobs(16, (3, 64, 64), 10, seed=1), class_blobs(16, (3, 64, 64), 10, seed=2), 10
        workers = 0
    else:
        tf = torchvision.models.ResNet18_Weights.IMAGENET1K_V1.transforms()
        calib = torchvision.datasets.ImageFolder(f"{args.data_root}/train", tf)
        val = torchvision.datasets.ImageFolder(f"{args.data_root}/val", tf)
        g = torch.Generator().manual_seed(args.seed)
        calib = Subset(calib, torch.randperm(len(calib), generator=g)[: args.calib_samples].tolist())
        if args.eval_samples:
            val = Subset(val, torch.randperm(len(val), generator=g)[: args.eval_samples].tolist())
        classes, workers = 1000, args.num_workers
    calib_loader = DataLoader(calib, args.batch_size, shuffle=False, num_workers=workers)
    val_loader = DataLoader(val, args.batch_size, shuffle=False, num_workers=workers)
    ann = torchvision.models.resnet18(weights=None if args.synthetic else args.weights, num_classes=classes).to(device).eval()
    results = {"ann": evaluate_ann(ann, val_loader, device), "snn": {}}
    makers = {"rate_max": lambda: ann2snn.RateCodingRecipe(dataloader=calib_loader, mode="max"),
              "rate_99.9%": lambda: ann2snn.RateCodingRecipe(dataloader=calib_loader, mode="99.9%"),
              "ltb": lambda: ann2snn.LocalThresholdBalancingRecipe(dataloader=calib_loader)}
    for name in args.recipes:
        snn = ann2snn.Converter(recipe=makers[name](), device=device).convert(ann)
        delay = sum(isinstance(m, neuron.BaseNode) for m in snn.modules()) if args.delay_start == "auto" else int(args.delay_start)
        results["snn"][name] = {"delay_start": delay, **{f"T={T}": evaluate_snn(snn, val_loader, device, T, delay) for T in args.time_steps}}
    return report(results, args.output)


if __name__ == "__main__":
    main()
