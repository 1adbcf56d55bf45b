"""Measurement callbacks of the memory-optimisation example, for the plain training loop in ``train.py`` (the reference's
``examples/memopt/lightning_callbacks.py`` hooks into Lightning's trainer; the hook names are kept).  Every figure is global:
per-rank sums are added over the process group before dividing, so two ranks that each spend 200 ms on 2 batches report
100 ms per batch.

Hooks receive ``(trainer, module, ...)``; ``trainer`` offers ``is_global_zero``, ``max_epochs``, ``current_epoch`` and ``device``."""
import time

import torch
import torch.distributed as dist


class Callback:
    def on_fit_start(self, trainer, module): pass
    def on_train_epoch_start(self, trainer, module): pass
    def on_train_batch_start(self, trainer, module, batch, batch_idx): pass
    def on_train_batch_end(self, trainer, module, outputs, batch, batch_idx): pass
    def on_train_epoch_end(self, trainer, module): pass
    def on_validation_epoch_start(self, trainer, module): pass
    def on_validation_batch_start(self, trainer, module, batch, batch_idx): pass
    def on_validation_batch_end(self, trainer, module, outputs, batch, batch_idx): pass
    def on_validation_epoch_end(self, trainer, module): pass
    def state_dict(self): return {}
    def load_state_dict(self, sd): pass


def _global_sum(values, device):
    """Element-wise sum of ``values`` over all ranks (the values themselves without a process group)."""
    if not (dist.is_available() and dist.is_initialized()):
        return list(values)
    t = torch.tensor(list(values), dtype=torch.float64, device=device if dist.get_backend() == "nccl" else "cpu")
    dist.all_reduce(t)
    return t.tolist()


def _say(trainer, text):
    if trainer.is_global_zero:
        print(f"Epoch {trainer.current_epoch}/{trainer.max_epochs}: {text}")


class _PhaseTotals(Callback):
    """Two running totals per phase (train / val), reduced over ranks at the end of an epoch."""
    fields = ("a", "b")

    def __init__(self, reset_per_epoch: bool = True):
        self.reset_per_epoch = reset_per_epoch
        self.totals = {"train": [0.0, 0.0], "val": [0.0, 0.0]}
        self.last = {}

    def _finish(self, trainer, phase):
        a, b = _global_sum(self.totals[phase], trainer.device)
        if self.reset_per_epoch:
            self.totals[phase] = [0.0, 0.0]
        return a, b

    def state_dict(self):
        return {"totals": {k: list(v) for k, v in self.totals.items()}, "reset_per_epoch": self.reset_per_epoch}

    def load_state_dict(self, sd):
        self.totals = {k: list(v) for k, v in sd["totals"].items()}
        self.reset_per_epoch = sd["reset_per_epoch"]


class GlobalMeanBatchTimeCallback(_PhaseTotals):
    """Mean wall time of a batch: (sum over ranks of time spent in batches) / (sum over ranks of batch counts)."""

    def __init__(self, reset_per_epoch: bool = False):
        super().__init__(reset_per_epoch)
        self._t0 = 0.0

    def _start(self):
        self._t0 = time.time()

    def _stop(self, phase):
        self.totals[phase][0] += time.time() - self._t0
        self.totals[phase][1] += 1

    def on_train_batch_start(self, *a, **k): self._start()
    def on_validation_batch_start(self, *a, **k): self._start()
    def on_train_batch_end(self, *a, **k): self._stop("train")
    def on_validation_batch_end(self, *a, **k): self._stop("val")

    def _report(self, trainer, phase):
        total, n = self._finish(trainer, phase)
        self.last[phase] = total / n if n > 0 else 0.0
        _say(trainer, f"global_mean_{phase}_batch_time={self.last[phase] * 1000:.2f} ms")

    def on_train_epoch_end(self, trainer, module): self._report(trainer, "train")
    def on_validation_epoch_end(self, trainer, module): self._report(trainer, "val")


class SamplePerSecondCallback(_PhaseTotals):
    """Samples per second of an epoch: samples summed over ranks, divided by the longest rank's epoch time."""

    def __init__(self, batch_size=None):
        super().__init__(True)
        self.batch_size = batch_size
        self._t0 = {"train": 0.0, "val": 0.0}

    def _count(self, phase, batch):
        first = batch[0] if isinstance(batch, (tuple, list)) else batch
        self.totals[phase][0] += self.batch_size if self.batch_size is not None else first.shape[0]

    def on_train_epoch_start(self, *a, **k): self._t0["train"] = time.time()
    def on_validation_epoch_start(self, *a, **k): self._t0["val"] = time.time()
    def on_train_batch_end(self, trainer, module, outputs, batch, batch_idx): self._count("train", batch)
    def on_validation_batch_end(self, trainer, module, outputs, batch, batch_idx): self._count("val", batch)

    def _report(self, trainer, phase):
        elapsed = time.time() - self._t0[phase]
        if dist.is_available() and dist.is_initialized():
            t = torch.tensor([elapsed], dtype=torch.float64, device=trainer.device if dist.get_backend() == "nccl" else "cpu")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            elapsed = float(t)
        samples, _ = self._finish(trainer, phase)
        self.last[phase] = samples / elapsed if elapsed > 0 else 0.0
        _say(trainer, f"{phase}_samples_per_second={self.last[phase]:.1f}")

    def on_train_epoch_end(self, trainer, module): self._report(trainer, "train")
    def on_validation_epoch_end(self, trainer, module): self._report(trainer, "val")


class PeakMemoryTillNowCallback(Callback):
    """Peak allocated device memory since the start of the fit, the largest over ranks."""

    def __init__(self):
        self.peak_mb = 0.0

    def on_fit_start(self, trainer, module):
        if trainer.device.type == "cuda":
            torch.cuda.reset_peak_memory_stats(trainer.device)

    def on_train_epoch_end(self, trainer, module):
        if trainer.device.type != "cuda":
            return
        peak = torch.cuda.max_memory_allocated(trainer.device) / 2 ** 20
        if dist.is_available() and dist.is_initialized():
            t = torch.tensor([peak], dtype=torch.float64, device=trainer.device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            peak = float(t)
        self.peak_mb = peak
        _say(trainer, f"peak_memory_till_now={peak:.1f} MB")

    def state_dict(self): return {"peak_mb": self.peak_mb}
    def load_state_dict(self, sd): self.peak_mb = sd["peak_mb"]
