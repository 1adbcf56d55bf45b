"""Config-driven single-node trainer of the CIFAR10-DVS VGG with automatic memory optimisation (the role of the reference's
``examples/memopt/train.py``, which builds the same objects through LightningCLI; this one reads the same kind of YAML --
``class_path`` / ``init_args`` entries -- and runs a plain loop with the hooks of ``callbacks.py``):

    python -m spikingjelly_b200.activation_based.examples.memopt.train --config config.yaml --set data.synthetic=true trainer.max_epochs=1

The network goes through ``memopt.memory_optimization(net, (VGGBlock,), dummy_input, compress_x, level)`` before training, the
best validation accuracy keeps a checkpoint, and every epoch appends a row to ``metrics.csv`` under ``default_root_dir``.
"""
import argparse
import contextlib
import csv
import importlib
import random
from pathlib import Path

import numpy as np
import torch
import yaml

from ... import memopt
from .callbacks import GlobalMeanBatchTimeCallback, PeakMemoryTillNowCallback, SamplePerSecondCallback
from .data_module import CIFAR10DVSDataModule
from .models import VGGBlock
from .modules import ClassificationModule

DEFAULT_CONFIG = Path(__file__).with_name("config.yaml")


def instantiate(spec, *args, **extra):
    """``{class_path, init_args}`` -> object, recursively; anything else is returned as it is."""
    if not (isinstance(spec, dict) and "class_path" in spec):
        return spec
    module, _, name = spec["class_path"].rpartition(".")
    kwargs = {k: instantiate(v) for k, v in (spec.get("init_args") or {}).items()}
    return getattr(importlib.import_module(module), name)(*args, **kwargs, **extra)


def override(config: dict, assignments):
    """``a.b.c=value`` assignments (values parsed as YAML) applied to the nested dictionary."""
    for item in assignments or ():
        path, _, raw = item.partition("=")
        node, keys = config, path.split(".")
        for k in keys[:-1]:
            node = node.setdefault(k, {})
        node[keys[-1]] = yaml.safe_load(raw)
    return config


class Trainer:
    def __init__(self, max_epochs: int, device: torch.device, precision="32", root: Path = Path("."), callbacks=(), max_steps: int = 0):
        self.max_epochs, self.device, self.precision, self.root = max_epochs, device, str(precision), Path(root)
        self.callbacks, self.max_steps, self.current_epoch, self.is_global_zero = list(callbacks), max_steps, 0, True
        self.history, self.best_acc = [], -1.0

    def _call(self, hook, *args):
        for cb in self.callbacks:
            getattr(cb, hook)(self, *args)

    def _autocast(self):
        if self.precision in ("bf16", "bf16-mixed") and self.device.type == "cuda":
            return torch.autocast("cuda", dtype=torch.bfloat16)
        return contextlib.nullcontext()

    def _to_device(self, batch):
        return tuple(b.to(self.device, non_blocking=True) for b in batch)

    def fit(self, module, datamodule, optimizer, scheduler=None):
        datamodule.prepare_data()
        datamodule.setup("fit")
        self.root.mkdir(parents=True, exist_ok=True)
        self._call("on_fit_start", module)
        for epoch in range(self.max_epochs):
            self.current_epoch = epoch
            module.train()
            self._call("on_train_epoch_start", module)
            for i, batch in enumerate(datamodule.train_dataloader()):
                if self.max_steps and i >= self.max_steps:
                    break
                batch = self._to_device(batch)
                self._call("on_train_batch_start", module, batch, i)
                optimizer.zero_grad(set_to_none=True)
                with self._autocast():
                    loss = module.training_step(batch, i)
                loss.backward()
                optimizer.step()
                self._call("on_train_batch_end", module, loss.detach(), batch, i)
            train = module.epoch_summary("train")
            self._call("on_train_epoch_end", module)
            module.eval()
            self._call("on_validation_epoch_start", module)
            for i, batch in enumerate(datamodule.val_dataloader()):
                if self.max_steps and i >= self.max_steps:
                    break
                batch = self._to_device(batch)
                self._call("on_validation_batch_start", module, batch, i)
                with self._autocast():
                    loss = module.validation_step(batch, i)
                self._call("on_validation_batch_end", module, loss, batch, i)
            val = module.epoch_summary("val")
            self._call("on_validation_epoch_end", module)
            if scheduler is not None:
                scheduler.step()
            row = {"epoch": epoch, "train_loss": train["loss"], "train_acc": train["acc"], "val_loss": val["loss"], "val_acc": val["acc"],
                   "lr": optimizer.param_groups[0]["lr"]}
            self.history.append(row)
            print(f"Epoch {epoch}/{self.max_epochs}: train_loss={train['loss']:.2f}, train_acc={train['acc']:.2f}%, "
                  f"val_loss={val['loss']:.2f}, val_acc={val['acc']:.2f}%")
            with open(self.root / "metrics.csv", "a", newline="") as f:
                w = csv.DictWriter(f, fieldnames=list(row))
                if f.tell() == 0:
                    w.writeheader()
                w.writerow(row)
            if val["acc"] > self.best_acc:
                self.best_acc = val["acc"]
                torch.save({"epoch": epoch, "net": module.net.state_dict(), "optimizer": optimizer.state_dict(), "val_acc": val["acc"],
                            "callbacks": {type(cb).__name__: cb.state_dict() for cb in self.callbacks}}, self.root / "best.pt")
        return self.history


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=Path, default=DEFAULT_CONFIG)
    ap.add_argument("--set", nargs="*", default=[], metavar="KEY=VALUE", help="overrides, e.g. data.synthetic=true trainer.max_epochs=1")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--max-steps", type=int, default=0, help="stop every epoch after this many batches (0: whole epoch)")
    a = ap.parse_args(argv)
    cfg = override(yaml.safe_load(a.config.read_text()), a.set)
    seed = int(cfg.get("seed_everything", 0))
    random.seed(seed), np.random.seed(seed), torch.manual_seed(seed)
    device = torch.device(a.device)
    m, d, t = cfg["model"], cfg["data"], cfg.get("trainer", {})
    if m["T"] != d["T"]:
        raise ValueError(f"model.T ({m['T']}) and data.T ({d['T']}) differ")
    if device.type != "cuda":                       # the kernel backend needs a GPU; the same model runs eagerly on the host
        m["net"].setdefault("init_args", {})["backend"] = "torch"
    data = CIFAR10DVSDataModule(**d)
    net = instantiate(m["net"]).to(device)
    res = getattr(net, "resolution", data.resolution)
    net = memopt.memory_optimization(net, (VGGBlock,), dummy_input=(torch.zeros(d["batch_size"], m["T"], 2, res, res, device=device),),
                                     compress_x=bool(m.get("compress_x", False)), level=int(m.get("level", 0))).to(device)   # it comes back on the host
    module = ClassificationModule(net, instantiate(m["criterion"]), num_classes=10, y_with_T=True).to(device)
    optimizer = instantiate(cfg["optimizer"], module.parameters())
    scheduler = instantiate(cfg["lr_scheduler"], optimizer) if cfg.get("lr_scheduler") else None
    trainer = Trainer(int(t.get("max_epochs", 1)), device, t.get("precision", "32"), Path(t.get("default_root_dir", "./logs/CIFAR10DVS")),
                      [GlobalMeanBatchTimeCallback(reset_per_epoch=True), SamplePerSecondCallback(), PeakMemoryTillNowCallback()], a.max_steps)
    return trainer.fit(module, data, optimizer, scheduler)


if __name__ == "__main__":
    main()
