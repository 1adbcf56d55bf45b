#!/usr/bin/env python
"""ANN (no spiking neuron) training under each precision policy, through the public precision API: forward, backward and
optimizer time per step, samples/s and peak memory.  One script for the three GEMM-heavy workloads the reference times in
``benchmark/benchmark_train_precision_ann_single_linear.py`` (one 8192 x 8192 linear, batch 32768),
``..._ann_linear_only.py`` (32 x [Linear(2048) + GELU], batch 8192) and ``..._ann_attention.py`` (24 residual MLP blocks of
width 2048 with an attention block after every fourth, batch 256 x 128 tokens).

    python benchmark/benchmark_train_precision_ann.py --model single_linear|linear_only|attention [--precisions fp32 bf16 fp8]
        [--impl ours|reference]
"""
import argparse
import json
import statistics
import sys
from pathlib import Path

import torch
import torch.nn as nn
import torch.nn.functional as F

sys.path.insert(0, str(Path(__file__).resolve().parent))
import _arms  # noqa: E402

DEFAULTS = {
    "single_linear": dict(batch_size=32768, input_dim=8192, hidden_dim=0, num_classes=8192, depth=1),
    "linear_only": dict(batch_size=8192, input_dim=2048, hidden_dim=2048, num_classes=2048, depth=32),
    "attention": dict(batch_size=256, input_dim=1024, hidden_dim=2048, num_classes=1024, depth=24),
}


class LinearStack(nn.Module):
    def __init__(self, input_dim, hidden_dim, num_classes, depth):
        super().__init__()
        mods, width = [], input_dim
        for _ in range(depth - 1):
            mods += [nn.Linear(width, hidden_dim), nn.GELU()]
            width = hidden_dim
        self.net = nn.Sequential(*mods, nn.Linear(width, num_classes))

    def forward(self, x):
        return self.net(x)


class MLPBlock(nn.Module):
    def __init__(self, dim, ratio=4):
        super().__init__()
        self.net = nn.Sequential(nn.LayerNorm(dim), nn.Linear(dim, dim * ratio), nn.GELU(), nn.Linear(dim * ratio, dim))

    def forward(self, x):
        return x + self.net(x)


class AttentionBlock(nn.Module):
    def __init__(self, dim, heads, ratio=4):
        super().__init__()
        self.norm1, self.norm2, self.heads = nn.LayerNorm(dim), nn.LayerNorm(dim), heads
        self.q_proj, self.k_proj, self.v_proj, self.out_proj = (nn.Linear(dim, dim) for _ in range(4))
        self.mlp = nn.Sequential(nn.Linear(dim, dim * ratio), nn.GELU(), nn.Linear(dim * ratio, dim))

    def forward(self, x):
        b, t, c = x.shape
        y = self.norm1(x)
        q, k, v = (p(y).view(b, t, self.heads, c // self.heads).transpose(1, 2) for p in (self.q_proj, self.k_proj, self.v_proj))
        x = x + self.out_proj(F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(b, t, c))
        return x + self.mlp(self.norm2(x))


class DeepANN(nn.Module):
    def __init__(self, input_dim, hidden_dim, num_classes, depth, attention_every, heads):
        super().__init__()
        self.token_proj = nn.Linear(input_dim, hidden_dim)
        self.blocks = nn.ModuleList()
        for i in range(depth):
            self.blocks.append(MLPBlock(hidden_dim))
            if attention_every > 0 and (i + 1) % attention_every == 0:
                self.blocks.append(AttentionBlock(hidden_dim, heads))
        self.head_norm, self.head = nn.LayerNorm(hidden_dim), nn.Linear(hidden_dim, num_classes)

    def forward(self, x):
        x = self.token_proj(x)
        for b in self.blocks:
            x = b(x)
        return self.head(self.head_norm(x.mean(dim=1)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--model", choices=sorted(DEFAULTS), default="linear_only")
    ap.add_argument("--precisions", nargs="+", default=None)
    for k in ("batch_size", "input_dim", "hidden_dim", "num_classes", "depth"):
        ap.add_argument("--" + k.replace("_", "-"), type=int, default=None)
    ap.add_argument("--seq-len", type=int, default=128)
    ap.add_argument("--attention-every", type=int, default=4)
    ap.add_argument("--num-heads", type=int, default=16)
    ap.add_argument("--lr", type=float, default=5e-2)
    ap.add_argument("--momentum", type=float, default=0.9)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--seed", type=int, default=20260531)
    ap.add_argument("--device", default="cuda:0")
    a = ap.parse_args()
    cfg = {k: (getattr(a, k) if getattr(a, k) is not None else v) for k, v in DEFAULTS[a.model].items()}
    try:
        arm = _arms.load(a.impl)
        precision = arm.get("precision")
    except Exception as exc:
        return _arms.unavailable(a.impl, exc)
    modes = a.precisions or (["fp32", "bf16", "fp8"] if a.impl == "ours" else ["fp32", "bf16", "fp8-torchao"])
    dev = torch.device(a.device)
    cuda = dev.type == "cuda"

    def build():
        torch.manual_seed(a.seed)
        if a.model == "attention":
            return DeepANN(cfg["input_dim"], cfg["hidden_dim"], cfg["num_classes"], cfg["depth"], a.attention_every, a.num_heads).to(dev)
        return LinearStack(cfg["input_dim"], cfg["hidden_dim"], cfg["num_classes"], cfg["depth"]).to(dev)
    shape = (cfg["batch_size"], a.seq_len, cfg["input_dim"]) if a.model == "attention" else (cfg["batch_size"], cfg["input_dim"])
    x = torch.randn(shape, device=dev)
    y = torch.randint(cfg["num_classes"], (cfg["batch_size"],), device=dev)
    for mode in modes:
        try:
            art = precision.prepare_model_for_precision(build(), dev, precision.PrecisionConfig(mode=mode, strictness="strict", device=str(dev)))
            net = art.model.train()
            opt = torch.optim.SGD(net.parameters(), lr=a.lr, momentum=a.momentum)
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)] if cuda else None
            parts, loss = {"forward_ms": [], "backward_ms": [], "optimizer_ms": [], "total_step_ms": []}, None
            if cuda:
                torch.cuda.reset_peak_memory_stats(dev)
            for i in range(a.warmup + a.steps):
                opt.zero_grad(set_to_none=True)
                if cuda:
                    ev[0].record()
                with art.autocast_context():
                    loss = F.cross_entropy(net(x).float(), y)
                if cuda:
                    ev[1].record()
                art.backward(loss, opt, step_optimizer=False)
                if cuda:
                    ev[2].record()
                opt.step()
                if cuda:
                    ev[3].record()
                    ev[3].synchronize()
                    if i >= a.warmup:
                        for name, (s, e) in zip(parts, ((0, 1), (1, 2), (2, 3), (0, 3))):
                            parts[name].append(ev[s].elapsed_time(ev[e]))
            row = {"impl": a.impl, "model": a.model, "precision": mode, **cfg, "loss": round(float(loss), 4)}
            if cuda:
                row.update({k: round(statistics.median(v), 3) for k, v in parts.items()})
                row["samples_per_s"] = round(cfg["batch_size"] / row["total_step_ms"] * 1e3, 1)
                row["peak_allocated_mb"] = round(torch.cuda.max_memory_allocated(dev) / 2 ** 20, 1)
            report = art.describe().get("conversion_report") if hasattr(art, "describe") else None
            if isinstance(report, dict):
                row["converted_modules"] = len(report.get("converted_modules") or [])
        except Exception as exc:
            row = {"impl": a.impl, "model": a.model, "precision": mode, "unavailable": f"{type(exc).__name__}: {exc}"[:200]}
        print(json.dumps(row, default=str), flush=True)
        del row
        if cuda:
            torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
