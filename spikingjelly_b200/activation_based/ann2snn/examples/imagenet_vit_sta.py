"""Vision transformer -> spiking transformer with the STA recipe: ``equivalent`` mode (time-difference operators, the accumulated
output equals the source network after every step) and ``spiking_encoder`` mode (integrate-and-fire re-encoding of the residual
stream with calibrated thresholds; accuracy approaches the source network as T grows).  torchvision ``vit_b_16`` on an ImageNet
folder, or a four-block ViT on generated images with ``--synthetic``.  Role of
``spikingjelly/activation_based/ann2snn/examples/imagenet_vit_sta.py``.

    python -m spikingjelly_b200.activation_based.ann2snn.examples.imagenet_vit_sta --synthetic --time-steps 8
"""
import argparse

import torch
import torch.nn as nn
from torch.utils.data import DataLoader, Subset

from ... import ann2snn, functional
from ._common import add_common_args, class_blobs, report


class Block(nn.Module):
    def __init__(self, dim, heads):
        super().__init__()
        self.norm1, self.attn, self.norm2 = nn.LayerNorm(dim), nn.MultiheadAttention(dim, heads, batch_first=True), nn.LayerNorm(dim)
        self.fc1, self.act, self.fc2 = nn.Linear(dim, 2 * dim), nn.GELU(), nn.Linear(2 * dim, dim)

    def forward(self, x):
        y = self.norm1(x)
        a, _ = self.attn(y, y, y, need_weights=False)
        x = x + a
        return x + self.fc2(self.act(self.fc1(self.norm2(x))))


class SmallViT(nn.Module):
    def __init__(self, image=32, patch=8, dim=64, heads=4, depth=4, classes=10):
        super().__init__()
        self.patch_size, self.embed = patch, nn.Linear(3 * patch * patch, dim)
        self.position = nn.Parameter(torch.zeros(1, (image // patch) ** 2, dim).normal_(std=0.02))
        self.blocks = nn.Sequential(*[Block(dim, heads) for _ in range(depth)])
        self.norm, self.head = nn.LayerNorm(dim), nn.Linear(dim, classes)

    def forward(self, x):                                  # [B, 3, H, W], or patch rows [B, L, 3 * p * p] (what the converted network is fed)
        if x.dim() == 4:
            x = patches(x, self.patch_size)
        return self.head(self.norm(self.blocks(self.embed(x) + self.position)).mean(-2))              # a negative axis: the converted graph runs on [T, B, L, C]


def patches(img: torch.Tensor, size: int) -> torch.Tensor:
    """Non-overlapping ``size x size`` patches as rows: ``[B, 3, H, W] -> [B, L, 3 * size * size]``."""
    return nn.functional.unfold(img, size, stride=size).transpose(1, 2)


class PatchRows(nn.Module):
    """The token part of :class:`SmallViT` (everything behind the patch extraction), the network that is converted."""

    def __init__(self, vit: SmallViT):
        super().__init__()
        self.embed, self.position, self.blocks, self.norm, self.head = vit.embed, vit.position, vit.blocks, vit.norm, vit.head

    def forward(self, x):
        return self.head(self.norm(self.blocks(self.embed(x) + self.position)).mean(-2))              # a negative axis: the converted graph runs on [T, B, L, C]


@torch.no_grad()
def evaluate(model, loader, device, time_steps=None, prepare=None):
    """Top-1 of the source network (``time_steps`` None) or of the converted one: the image is presented at the first step and
    zeros afterwards, the outputs of all steps are summed."""
    model.eval()
    hit = total = 0
    gap = 0.0
    for img, label in loader:
        img = img.to(device)
        if prepare is not None:
            img = prepare(img)
        if time_steps is None:
            out = model(img)
        else:
            functional.reset_net(model)
            seq = torch.zeros((time_steps,) + tuple(img.shape), device=device)
            seq[0] = img
            out = model(seq).sum(0)
        hit += int((out.argmax(1).cpu() == label).sum())
        total += label.numel()
    return hit / total


def main(argv=None):
    p = add_common_args(argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter))
    p.add_argument("--data-root", default=None)
    p.add_argument("--weights", default=None, help="torchvision weight name for vit_b_16, e.g. IMAGENET1K_V1")
    p.add_argument("--calib-samples", type=int, default=512)
    p.add_argument("--eval-samples", type=int, default=1000)
    p.add_argument("--batch-size", type=int, default=32)
    p.add_argument("--time-steps", type=int, default=32)
    p.add_argument("--modes", nargs="+", default=["equivalent", "spiking_encoder"], choices=["equivalent", "spiking_encoder"])
    p.add_argument("--threshold-mode", default="mse", choices=["mse", "max"])
    args = p.parse_args(argv)
    torch.manual_seed(args.seed)
    device = torch.device(args.device)
    if args.synthetic:
        calib, val = class_blobs(64, (3, 32, 32), 10, seed=1), class_blobs(64, (3, 32, 32), 10, seed=2)
        ann = SmallViT().to(device)
        from ._common import fit
        fit(ann, DataLoader(class_blobs(512, (3, 32, 32), 10, seed=3), 64, shuffle=True), device, epochs=3, lr=3e-3)
    else:
        import torchvision
        tf = torchvision.models.ViT_B_16_Weights.IMAGENET1K_V1.transforms()
        g = torch.Generator().manual_seed(args.seed)
        train, val = torchvision.datasets.ImageFolder(f"{args.data_root}/train", tf), torchvision.datasets.ImageFolder(f"{args.data_root}/val", tf)
        calib = Subset(train, torch.randperm(len(train), generator=g)[: args.calib_samples].tolist())
        val = Subset(val, torch.randperm(len(val), generator=g)[: args.eval_samples].tolist())
        ann = torchvision.models.vit_b_16(weights=args.weights).to(device)
    ann.eval()
    prepare = None
    if args.synthetic:                                     # convert the token network; patch extraction stays outside
        size = ann.patch_size
        ann, prepare = PatchRows(ann).eval(), (lambda img: patches(img, size))
        calib = [(patches(torch.stack([calib[i][0] for i in range(len(calib))]), size), torch.zeros(len(calib)))]
    calib_loader, val_loader = (calib if args.synthetic else DataLoader(calib, args.batch_size)), DataLoader(val, args.batch_size)
    results = {"time_steps": args.time_steps, "ann_top1": evaluate(ann, val_loader, device, prepare=prepare), "snn": {}}
    for mode in args.modes:
        recipe = ann2snn.STATransformerRecipe(dataloader=calib_loader, time_steps=args.time_steps, mode=mode, threshold_mode=args.threshold_mode)
        snn = ann2snn.Converter(recipe=recipe, device=device).convert(ann)
        results["snn"][mode] = {"top1": evaluate(snn, val_loader, device, args.time_steps, prepare)}
    return report(results, args.output)


if __name__ == "__main__":
    main()
