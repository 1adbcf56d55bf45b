"""Classification wrapper of the memory-optimisation example: loss on the raw network output (per-step logits when
``y_with_T``), accuracy on the time-averaged logits, running means per epoch (the reference's
``examples/memopt/lightning_modules.py`` without the Lightning and torchmetrics base classes)."""
import torch
import torch.nn as nn

from ... import functional


class _Mean:
    def __init__(self):
        self.total, self.n = 0.0, 0

    def update(self, value, n=1):
        self.total += float(value) * n
        self.n += n

    def compute(self):
        return self.total / max(self.n, 1)

    def reset(self):
        self.total, self.n = 0.0, 0


class ClassificationModule(nn.Module):
    def __init__(self, net: nn.Module, criterion: nn.Module, num_classes: int, y_with_T: bool = False):
        super().__init__()
        self.net, self.criterion, self.num_classes, self.y_with_T = net, criterion, num_classes, y_with_T
        self.metrics = {p: {"loss": _Mean(), "acc": _Mean()} for p in ("train", "val")}

    def forward(self, x):
        return self.net(x)

    def _step(self, batch, phase):
        x, label = batch[0].float(), batch[1]
        y = self(x)
        loss = self.criterion(y, label)
        functional.reset_net(self.net)
        if self.y_with_T:
            y = y.mean(dim=0)
        if label.ndim > 1:
            label = label.argmax(dim=1)
        n = label.shape[0]
        self.metrics[phase]["loss"].update(loss.detach(), n)
        self.metrics[phase]["acc"].update((y.argmax(dim=1) == label).float().mean(), n)
        return loss

    def training_step(self, batch, batch_idx):
        return self._step(batch, "train")

    @torch.no_grad()
    def validation_step(self, batch, batch_idx):
        return self._step(batch, "val")

    def epoch_summary(self, phase):
        """``{loss, acc}`` of the finished epoch (accuracy in percent); resets the running means."""
        out = {k: m.compute() * (100.0 if k == "acc" else 1.0) for k, m in self.metrics[phase].items()}
        for m in self.metrics[phase].values():
            m.reset()
        return out
