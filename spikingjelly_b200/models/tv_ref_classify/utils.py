"""Meters, distributed helpers and checkpoint utilities used by :class:`~spikingjelly_b200.models.train_classify.Trainer`.

Parity: ``spikingjelly/activation_based/model/tv_ref_classify/utils.py:26-698`` (same names and
semantics).  Meters accept tensors as well as Python numbers; tensors are accumulated on their
device without a host synchronisation and only read when a meter is printed or reduced.
"""
from __future__ import annotations

import copy
import datetime
import errno
import hashlib
import os
import time
from collections import OrderedDict, defaultdict, deque
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ...logger import logger

__all__ = ["SmoothedValue", "ThroughputValue", "MetricLogger", "ExponentialMovingAverage", "accuracy", "mkdir",
           "is_dist_avail_and_initialized", "get_world_size", "get_rank", "is_main_process", "save_on_master",
           "init_distributed_mode", "average_checkpoints", "store_model_weights", "reduce_across_processes"]


def _num(x) -> float:
    return float(x.item()) if torch.is_tensor(x) else float(x)


def is_dist_avail_and_initialized() -> bool:
    return dist.is_available() and dist.is_initialized()


def get_world_size() -> int:
    return dist.get_world_size() if is_dist_avail_and_initialized() else 1


def get_rank() -> int:
    return dist.get_rank() if is_dist_avail_and_initialized() else 0


def is_main_process() -> bool:
    return get_rank() == 0


def _reduce_device() -> torch.device:
    if is_dist_avail_and_initialized() and dist.get_backend() == "nccl":
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def reduce_across_processes(val, op=None, dtype=None):
    """Sum (default) of a scalar / tensor over all ranks; a plain tensor without a process group.  ``dtype``: dtype of the result."""
    if not is_dist_avail_and_initialized():
        return torch.as_tensor(val, dtype=dtype)
    t = torch.as_tensor(val, dtype=dtype, device=_reduce_device())
    dist.barrier()
    dist.all_reduce(t, op=op if op is not None else dist.ReduceOp.SUM)
    return t


class SmoothedValue:
    """Window of recent values plus running total; ``fmt`` may use median, avg, global_avg, max, value."""

    def __init__(self, window_size: int = 20, fmt: Optional[str] = None):
        self.deque = deque(maxlen=window_size)
        self.total, self.count = 0.0, 0
        self.fmt = fmt or "{median:.4f} ({global_avg:.4f})"

    def update(self, value, n: int = 1):
        self.deque.append(value)
        self.count += n
        self.total = self.total + value * n

    def synchronize_between_processes(self):
        """Only ``count`` and ``total`` are reduced; the window stays local."""
        t = reduce_across_processes([float(self.count), _num(self.total)]).tolist()
        self.count, self.total = int(t[0]), t[1]

    def _window(self) -> torch.Tensor:
        return torch.tensor([_num(v) for v in self.deque], dtype=torch.float32)

    @property
    def median(self):
        return self._window().median().item()

    @property
    def avg(self):
        return self._window().mean().item()

    @property
    def global_avg(self):
        return _num(self.total) / max(self.count, 1)

    @property
    def max(self):
        return max(_num(v) for v in self.deque)

    @property
    def value(self):
        return _num(self.deque[-1])

    def __str__(self):
        return self.fmt.format(median=self.median, avg=self.avg, global_avg=self.global_avg, max=self.max, value=self.value)


class ThroughputValue:
    """samples / elapsed seconds; the global average is total samples over total time, and after
    ``synchronize_between_processes`` the ranks' rates are added (they run concurrently)."""

    def __init__(self, window_size: int = 20, fmt: Optional[str] = None):
        self.deque = deque(maxlen=window_size)
        self.samples, self.elapsed = 0.0, 0.0
        self._synced_rate = None
        self.fmt = fmt or "{median:.1f} ({global_avg:.1f})"

    def update(self, samples, elapsed_time):
        self.deque.append(samples / max(elapsed_time, 1e-12))
        self.samples += samples
        self.elapsed += elapsed_time

    def synchronize_between_processes(self):
        self._synced_rate = float(reduce_across_processes(self.samples / max(self.elapsed, 1e-12)).item())

    @property
    def median(self):
        return torch.tensor(list(self.deque)).median().item() if self.deque else 0.0

    @property
    def avg(self):
        return torch.tensor(list(self.deque)).mean().item() if self.deque else 0.0

    @property
    def global_avg(self):
        if self._synced_rate is not None:
            return self._synced_rate
        return self.samples / max(self.elapsed, 1e-12)

    @property
    def max(self):
        return max(self.deque) if self.deque else 0.0

    @property
    def value(self):
        return self.deque[-1] if self.deque else 0.0

    def __str__(self):
        return self.fmt.format(median=self.median, avg=self.avg, global_avg=self.global_avg, max=self.max, value=self.value)


class MetricLogger:
    def __init__(self, delimiter: str = "\t"):
        self.meters = defaultdict(SmoothedValue)
        self.delimiter = delimiter

    def update(self, **kwargs):
        for k, v in kwargs.items():
            assert torch.is_tensor(v) or isinstance(v, (float, int))
            self.meters[k].update(v)

    def __getattr__(self, attr):
        meters = self.__dict__.get("meters", {})
        if attr in meters:
            return meters[attr]
        raise AttributeError(f"'{type(self).__name__}' object has no attribute '{attr}'")

    def __str__(self):
        return self.delimiter.join(f"{name}: {meter}" for name, meter in self.meters.items())

    def synchronize_between_processes(self):
        for meter in self.meters.values():
            meter.synchronize_between_processes()

    def add_meter(self, name, meter):
        self.meters[name] = meter

    def log_every(self, iterable, print_freq: int, header: Optional[str] = None):
        """Yield from ``iterable``; every ``print_freq`` items (never if <= 0) log progress, ETA,
        meters, iteration and data-loading time (and peak CUDA memory)."""
        header = header or ""
        n = len(iterable) if hasattr(iterable, "__len__") else None
        iter_time, data_time = SmoothedValue(fmt="{avg:.4f}"), SmoothedValue(fmt="{avg:.4f}")
        start = end = time.time()
        for i, obj in enumerate(iterable):
            data_time.update(time.time() - end)
            yield obj
            iter_time.update(time.time() - end)
            if print_freq > 0 and i % print_freq == 0:
                parts = [header, f"[{i}/{n}]" if n is not None else f"[{i}]"]
                if n is not None:
                    parts.append("eta: " + str(datetime.timedelta(seconds=int(iter_time.global_avg * (n - i)))))
                parts += [str(self), f"time: {iter_time}", f"data: {data_time}"]
                if torch.cuda.is_available():
                    parts.append(f"max mem: {torch.cuda.max_memory_allocated() / (1 << 20):.0f}")
                logger.info(self.delimiter.join(parts))
            end = time.time()
        logger.info("%s Total time: %s", header, datetime.timedelta(seconds=int(time.time() - start)))


class ExponentialMovingAverage(torch.optim.swa_utils.AveragedModel):
    """EMA of parameters *and* buffers: ``avg = decay * avg + (1 - decay) * value``."""

    def __init__(self, model, decay: float, device="cpu"):
        def ema(avg, value, num_averaged):
            return decay * avg + (1.0 - decay) * value
        super().__init__(model, device, ema, use_buffers=True)


def accuracy(output: torch.Tensor, target: torch.Tensor, topk: Tuple[int, ...] = (1,)) -> List[torch.Tensor]:
    """Top-k accuracies in percent (0-dim tensors on ``output``'s device).  Soft targets (mixup /
    cutmix) count as their arg-max class."""
    with torch.inference_mode():
        if target.ndim == 2:
            target = target.argmax(dim=1)
        k_max = min(max(topk), output.shape[1])
        pred = output.topk(k_max, dim=1).indices                    # [B, k]
        hits = pred.eq(target[:, None])
        return [hits[:, :min(k, k_max)].any(dim=1).float().mean() * 100.0 for k in topk]


def mkdir(path: str) -> None:
    try:
        os.makedirs(path)
    except OSError as e:
        if e.errno != errno.EEXIST:
            raise


def save_on_master(*args, **kwargs) -> None:
    if is_main_process():
        torch.save(*args, **kwargs)


def init_distributed_mode(args) -> None:
    """Fill ``args.rank / world_size / gpu / distributed`` from torchrun's or SLURM's environment and
    create the process group (NCCL on CUDA, gloo otherwise)."""
    if "RANK" in os.environ and "WORLD_SIZE" in os.environ:
        args.rank, args.world_size = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
        args.gpu = int(os.environ.get("LOCAL_RANK", 0))
    elif "SLURM_PROCID" in os.environ:
        args.rank = int(os.environ["SLURM_PROCID"])
        args.gpu = args.rank % max(torch.cuda.device_count(), 1)
    elif hasattr(args, "rank"):
        pass
    else:
        logger.info("Not using distributed mode")
        args.distributed = False
        return
    args.distributed = True
    use_cuda = torch.cuda.is_available() and str(getattr(args, "device", "cuda")).startswith("cuda")
    if use_cuda:
        torch.cuda.set_device(args.gpu)
    args.dist_backend = "nccl" if use_cuda else "gloo"
    logger.info("| distributed init (rank %s): %s", args.rank, args.dist_url)
    kwargs = dict(device_id=torch.device("cuda", args.gpu)) if use_cuda else {}
    dist.init_process_group(backend=args.dist_backend, init_method=args.dist_url, world_size=args.world_size,
                            rank=args.rank, **kwargs)
    dist.barrier()


def average_checkpoints(inputs: List[str]) -> OrderedDict:
    """Element-wise mean of the ``"model"`` state dicts stored in the checkpoint files ``inputs``;
    returns the first checkpoint with ``"model"`` replaced.  Key sets must agree."""
    summed, first, keys = OrderedDict(), None, None
    for path in inputs:
        state = torch.load(path, map_location="cpu", weights_only=False)
        first = first if first is not None else state
        model = state["model"]
        if keys is None:
            keys = list(model.keys())
        elif keys != list(model.keys()):
            raise KeyError(f"For checkpoint {path}, expected list of params: {keys}, but found: {list(model.keys())}")
        for k, v in model.items():
            v = v.float() if v.dtype == torch.float16 else v
            summed[k] = v.clone() if k not in summed else summed[k] + v
    averaged = OrderedDict()
    for k, v in summed.items():
        averaged[k] = v / len(inputs) if v.is_floating_point() else v // len(inputs)
    first["model"] = averaged
    return first


def store_model_weights(model, checkpoint_path: str, checkpoint_key: str = "model", strict: bool = True) -> str:
    """Extract the weights under ``checkpoint_key`` of a training checkpoint into
    ``weights-<sha256[:8]>.pth`` beside it (validated by loading them into a copy of ``model``)."""
    checkpoint_path = os.path.abspath(checkpoint_path)
    out_dir = os.path.dirname(checkpoint_path)
    model = copy.deepcopy(model)
    state = torch.load(checkpoint_path, map_location="cpu", weights_only=False)
    weights = state[checkpoint_key]
    if checkpoint_key == "model_ema":                      # AveragedModel prefixes and counts
        weights = {k[len("module."):]: v for k, v in weights.items() if k.startswith("module.")}
    model.load_state_dict(weights, strict=strict)
    tmp = os.path.join(out_dir, str(model.__hash__()))
    torch.save(model.state_dict(), tmp)
    sha = hashlib.sha256()
    with open(tmp, "rb") as f:
        for chunk in iter(lambda: f.read(4096), b""):
            sha.update(chunk)
    final = os.path.join(out_dir, "weights-" + sha.hexdigest()[:8] + ".pth")
    os.replace(tmp, final)
    return final
