"""Classification trainer: argument parser, data loading (ImageNet folder / CIFAR-10), optimiser and
schedule factories, AMP, EMA, mixup / cutmix, checkpoint + resume, TensorBoard, distributed data
parallel — with the hook methods a subclass overrides to plug in its network:

    class MyTrainer(Trainer):
        def load_model(self, args, num_classes): ...
        def preprocess_train_sample(self, args, x): ...    # e.g. repeat over T
        def process_model_output(self, args, y): ...       # e.g. mean over T

    trainer = MyTrainer(); trainer.main(trainer.get_args_parser().parse_args())

Parity: ``spikingjelly/activation_based/model/train_classify.py:32-1219`` (same arguments, hooks,
checkpoint keys ``model / optimizer / lr_scheduler / epoch / args / max_test_acc1 [/ model_ema /
max_ema_test_acc1 / scaler]`` and directory naming).  Differences by design: loss and accuracies are
accumulated on the device and read once per epoch (no host synchronisation per step); on CUDA the
multi-GPU wrapper is :class:`~spikingjelly_b200.parallel.data_parallel.SNNDataParallel` (fused NVLink
gradient all-reduce); autocast uses bf16, which needs no gradient scaler, unless ``--amp-dtype fp16``.
"""
from __future__ import annotations

import argparse
import datetime
import hashlib
import os
import random
import shutil
import sys
import time
import warnings

import numpy as np
import torch
import torch.utils.data
from torch import nn

from ..activation_based import functional
from ..logger import logger
from .tv_ref_classify import utils

__all__ = ["Trainer", "set_deterministic", "seed_worker"]


def set_deterministic(_seed_: int = 2020, disable_uda: bool = False) -> None:
    """Seed python / numpy / torch (all devices), make cuDNN deterministic and — unless
    ``disable_uda`` — switch on ``torch.use_deterministic_algorithms`` (with the cuBLAS workspace
    setting it requires)."""
    random.seed(_seed_)
    np.random.seed(_seed_)
    torch.manual_seed(_seed_)
    torch.cuda.manual_seed_all(_seed_)
    torch.backends.cudnn.deterministic = True
    torch.backends.cudnn.benchmark = False
    if not disable_uda:
        os.environ["CUBLAS_WORKSPACE_CONFIG"] = ":4096:8"
        torch.use_deterministic_algorithms(True)


def seed_worker(worker_id) -> None:
    """``worker_init_fn`` for DataLoader: derive numpy / random seeds from torch's per-worker seed."""
    seed = torch.initial_seed() % 2 ** 32
    np.random.seed(seed)
    random.seed(seed)


class _EpochStats:
    """Sums kept on the device; one read at the end of the epoch."""

    def __init__(self, device):
        self.sums = torch.zeros(4, dtype=torch.float64, device=device)     # loss, acc1, acc5, samples

    def add(self, loss, acc1, acc5, n):
        self.sums += torch.stack([loss.detach().double() * n, acc1.double() * n, acc5.double() * n,
                                  torch.as_tensor(float(n), dtype=torch.float64, device=self.sums.device)])

    def result(self):
        total = utils.reduce_across_processes(self.sums.clone()) if utils.is_dist_avail_and_initialized() else self.sums
        loss, a1, a5, n = total.tolist()
        n = max(n, 1.0)
        return loss / n, a1 / n, a5 / n, int(n)


class Trainer:
    # ------------------------------------------------------------------ hooks
    def get_data_to_device_kwargs(self, args):
        return {"non_blocking": not args.disable_pinmemory}

    def cal_acc1_acc5(self, output, target):
        return utils.accuracy(output, target, topk=(1, 5))

    def preprocess_train_sample(self, args, x: torch.Tensor):
        return x

    def preprocess_test_sample(self, args, x: torch.Tensor):
        return x

    def process_model_output(self, args, y: torch.Tensor):
        return y

    def before_train_one_epoch(self, args, model, epoch):
        pass

    def before_test_one_epoch(self, args, model, epoch):
        pass

    def load_model(self, args, num_classes):
        raise NotImplementedError("Users should define this function to load model")

    def load_data(self, args):
        return self.load_ImageNet(args)

    # ---------------------------------------------------------------- compile
    def compile_model(self, args, model: nn.Module, *, enabled=None) -> nn.Module:
        """Optional ``torch.compile`` (``--compile``); the native kernels do not depend on it."""
        enabled = args.compile if enabled is None else enabled
        if not enabled:
            return model
        kwargs = {"backend": args.compile_backend}
        if args.compile_mode is not None:
            kwargs["mode"] = args.compile_mode
        if args.compile_backend == "inductor" and args.compile_disable_cudagraphs:
            kwargs["options"] = {"triton.cudagraphs": False, "triton.cudagraph_trees": False}
        return torch.compile(model, **kwargs)

    def get_eval_model(self, args, train_model, model_without_ddp):
        return model_without_ddp if (args.compile and not args.compile_eval) else train_model

    # ------------------------------------------------------------------- AMP
    @staticmethod
    def _autocast(args, device):
        if args.disable_amp or device.type != "cuda":
            return torch.autocast(device.type, enabled=False)
        dtype = torch.float16 if getattr(args, "amp_dtype", "bf16") == "fp16" else torch.bfloat16
        return torch.autocast("cuda", dtype=dtype)

    # ------------------------------------------------------------------ loops
    def train_one_epoch(self, model, criterion, optimizer, data_loader, device, epoch, args, model_ema=None, scaler=None):
        model.train()
        stats = _EpochStats(device)
        to_dev = self.get_data_to_device_kwargs(args)
        t_epoch, seen = time.time(), 0
        for i, (image, target) in enumerate(data_loader):
            image, target = image.to(device, **to_dev), target.to(device, **to_dev)
            with self._autocast(args, device):
                image = self.preprocess_train_sample(args, image)
                output = self.process_model_output(args, model(image))
                loss = criterion(output, target)
            optimizer.zero_grad(set_to_none=True)
            if scaler is not None:
                scaler.scale(loss).backward()
                if args.clip_grad_norm is not None:
                    scaler.unscale_(optimizer)      # clip the true gradients
                    nn.utils.clip_grad_norm_(model.parameters(), args.clip_grad_norm)
                scaler.step(optimizer)
                scaler.update()
            else:
                loss.backward()
                if args.clip_grad_norm is not None:
                    nn.utils.clip_grad_norm_(model.parameters(), args.clip_grad_norm)
                optimizer.step()
            functional.reset_net(model)
            if model_ema and i % args.model_ema_steps == 0:
                model_ema.update_parameters(model)
                if epoch < args.lr_warmup_epochs:
                    model_ema.n_averaged.fill_(0)   # keep copying the weights during warm-up
            acc1, acc5 = self.cal_acc1_acc5(output, target)
            stats.add(loss, acc1, acc5, target.shape[0])
            seen += target.shape[0]
        train_loss, train_acc1, train_acc5, _ = stats.result()      # synchronises
        rate = seen * utils.get_world_size() / max(time.time() - t_epoch, 1e-9)
        if utils.is_main_process():
            logger.info("Train: train_acc1=%s, train_acc5=%s, train_loss=%s, samples/s=%s", train_acc1, train_acc5,
                        train_loss, rate)
        return train_loss, train_acc1, train_acc5

    def evaluate(self, args, model, criterion, data_loader, device, log_suffix=""):
        model.eval()
        stats = _EpochStats(device)
        to_dev = self.get_data_to_device_kwargs(args)
        start = time.time()
        with torch.inference_mode():
            for image, target in data_loader:
                image, target = image.to(device, **to_dev), target.to(device, **to_dev)
                image = self.preprocess_test_sample(args, image)
                output = self.process_model_output(args, model(image))
                loss = criterion(output, target)
                acc1, acc5 = self.cal_acc1_acc5(output, target)
                stats.add(loss, acc1, acc5, target.shape[0])
                functional.reset_net(model)
        test_loss, test_acc1, test_acc5, n = stats.result()
        if hasattr(data_loader.dataset, "__len__") and len(data_loader.dataset) != n and utils.is_main_process():
            warnings.warn(f"It looks like the dataset has {len(data_loader.dataset)} samples, but {n} samples were used for "
                          "the validation, which might bias the results. Try adjusting the batch size and / or the world "
                          "size. Setting the world size to 1 is always a safe bet.")
        if utils.is_main_process():
            logger.info("Test%s: test_acc1=%s, test_acc5=%s, test_loss=%s, samples/s=%s", f" {log_suffix}" if log_suffix else "",
                        test_acc1, test_acc5, test_loss, n / max(time.time() - start, 1e-9))
        return test_loss, test_acc1, test_acc5

    # ------------------------------------------------------------------- data
    def _get_cache_path(self, filepath):
        h = hashlib.sha1(filepath.encode()).hexdigest()
        return os.path.expanduser(os.path.join("~", ".torch", "vision", "datasets", "imagefolder", h[:10] + ".pt"))

    def _samplers(self, args, dataset, dataset_test):
        if args.distributed:
            if args.ra_sampler:
                from .tv_ref_classify.sampler import RASampler
                train_sampler = RASampler(dataset, shuffle=True, repetitions=args.ra_reps, seed=args.seed)
            else:
                train_sampler = torch.utils.data.distributed.DistributedSampler(dataset, seed=args.seed)
            return train_sampler, torch.utils.data.distributed.DistributedSampler(dataset_test, shuffle=False)
        g = torch.Generator()
        g.manual_seed(args.seed)
        return torch.utils.data.RandomSampler(dataset, generator=g), torch.utils.data.SequentialSampler(dataset_test)

    def load_CIFAR10(self, args):
        import torchvision
        from torchvision.transforms.functional import InterpolationMode
        from .tv_ref_classify import presets
        mean, std = (0.4914, 0.4822, 0.4465), (0.2023, 0.1994, 0.2010)
        dataset = torchvision.datasets.CIFAR10(root=args.data_path, train=True, transform=presets.ClassificationPresetTrain(
            crop_size=args.train_crop_size, mean=mean, std=std, interpolation=InterpolationMode(args.interpolation),
            auto_augment_policy=args.auto_augment, random_erase_prob=args.random_erase))
        dataset_test = torchvision.datasets.CIFAR10(root=args.data_path, train=False, transform=torchvision.transforms.Compose(
            [torchvision.transforms.ToTensor(), torchvision.transforms.Normalize(mean, std)]))
        return (dataset, dataset_test, *self._samplers(args, dataset, dataset_test))

    def load_ImageNet(self, args):
        import torchvision
        from torchvision.transforms.functional import InterpolationMode
        from .tv_ref_classify import presets
        interpolation = InterpolationMode(args.interpolation)

        def folder(split, transform):
            root = os.path.join(args.data_path, split)
            cache = self._get_cache_path(root)
            if args.cache_dataset and os.path.exists(cache):
                return torch.load(cache, weights_only=False)[0]     # the transforms are cached too
            ds = torchvision.datasets.ImageFolder(root, transform)
            if args.cache_dataset:
                utils.mkdir(os.path.dirname(cache))
                utils.save_on_master((ds, root), cache)
            return ds

        st = time.time()
        dataset = folder("train", presets.ClassificationPresetTrain(
            crop_size=args.train_crop_size, interpolation=interpolation, auto_augment_policy=args.auto_augment,
            random_erase_prob=args.random_erase))
        dataset_test = folder("val", presets.ClassificationPresetEval(
            crop_size=args.val_crop_size, resize_size=args.val_resize_size, interpolation=interpolation))
        if utils.is_main_process():
            logger.info("Datasets ready in %.1f s", time.time() - st)
        return (dataset, dataset_test, *self._samplers(args, dataset, dataset_test))

    # ------------------------------------------------------------- factories
    def get_tb_logdir_name(self, args):
        return (f"{args.model}_b{args.batch_size}_e{args.epochs}_{args.opt}_lr{args.lr}_wd{args.weight_decay}"
                f"_ls{args.label_smoothing}_ma{args.mixup_alpha}_ca{args.cutmix_alpha}_sbn{1 if args.sync_bn else 0}"
                f"_ra{args.ra_reps if args.ra_sampler else 0}_re{args.random_erase}_aaug{args.auto_augment}"
                f"_size{args.train_crop_size}_{args.val_resize_size}_{args.val_crop_size}_seed{args.seed}")

    def set_optimizer(self, args, parameters):
        name = args.opt.lower()
        if name.startswith("sgd"):
            return torch.optim.SGD(parameters, lr=args.lr, momentum=args.momentum, weight_decay=args.weight_decay,
                                   nesterov="nesterov" in name)
        if name == "rmsprop":
            return torch.optim.RMSprop(parameters, lr=args.lr, momentum=args.momentum, weight_decay=args.weight_decay,
                                       eps=0.0316, alpha=0.9)
        if name == "adamw":
            return torch.optim.AdamW(parameters, lr=args.lr, weight_decay=args.weight_decay)
        raise RuntimeError(f"Invalid optimizer {args.opt}. Only SGD, RMSprop and AdamW are supported.")

    def set_lr_scheduler(self, args, optimizer):
        args.lr_scheduler = args.lr_scheduler.lower()
        S = torch.optim.lr_scheduler
        main = {"step": lambda: S.StepLR(optimizer, step_size=args.lr_step_size, gamma=args.lr_gamma),
                "cosa": lambda: S.CosineAnnealingLR(optimizer, T_max=args.epochs - args.lr_warmup_epochs),
                "exp": lambda: S.ExponentialLR(optimizer, gamma=args.lr_gamma)}.get(args.lr_scheduler, lambda: None)()
        if args.lr_warmup_epochs <= 0:
            return main
        if args.lr_warmup_method == "linear":
            warm = S.LinearLR(optimizer, start_factor=args.lr_warmup_decay, total_iters=args.lr_warmup_epochs)
        elif args.lr_warmup_method == "constant":
            warm = S.ConstantLR(optimizer, factor=args.lr_warmup_decay, total_iters=args.lr_warmup_epochs)
        else:
            raise RuntimeError(f"Invalid warmup lr method '{args.lr_warmup_method}'. Only linear and constant are supported.")
        return S.SequentialLR(optimizer, schedulers=[warm, main], milestones=[args.lr_warmup_epochs])

    def _wrap_distributed(self, args, model, device):
        if device.type == "cuda":
            from ..parallel.data_parallel import prepare_snn_data_parallel
            return prepare_snn_data_parallel(model, device_ids=[args.gpu])
        return torch.nn.parallel.DistributedDataParallel(model)

    # ------------------------------------------------------------------ main
    def main(self, args):
        """Runs the whole job: set-up (:meth:`_set_up`), optional resume, then the epoch loop or a single evaluation."""
        run = self._set_up(args)
        if run is None:                       # --print-logdir
            return
        if args.resume is not None:
            self._resume(args, run)
        self._wrap_for_training(args, run)
        if args.test_only:
            target, tag = (run.model_ema, "EMA") if run.model_ema else (run.eval_model, "")
            self.evaluate(args, target, run.criterion, run.test_loader, device=run.device, log_suffix=tag)
            return
        for epoch in range(args.start_epoch, args.epochs):
            began = time.time()
            if args.distributed:
                run.train_sampler.set_epoch(epoch)
            self.before_train_one_epoch(args, run.model, epoch)
            loss, acc1, acc5 = self.train_one_epoch(run.model, run.criterion, run.optimizer, run.train_loader, run.device, epoch, args,
                                                    run.model_ema, run.scaler)
            if hasattr(run.model, "check_communication"):
                run.model.check_communication()        # a gradient exchange that gave up on a peer ends the job here
            run.log_scalars(epoch, train_loss=loss, train_acc1=acc1, train_acc5=acc5)
            if run.lr_scheduler is not None:
                run.lr_scheduler.step()
            self.before_test_one_epoch(args, run.eval_model, epoch)
            loss, acc1, acc5 = self.evaluate(args, run.eval_model, run.criterion, run.test_loader, device=run.device)
            run.log_scalars(epoch, test_loss=loss, test_acc1=acc1, test_acc5=acc5)
            ema_acc1 = None
            if run.model_ema:
                ema_loss, ema_acc1, ema_acc5 = self.evaluate(args, run.model_ema, run.criterion, run.test_loader, device=run.device,
                                                             log_suffix="EMA")
                run.log_scalars(epoch, ema_test_loss=ema_loss, ema_test_acc1=ema_acc1, ema_test_acc5=ema_acc5)
            self._save_checkpoints(args, run, epoch, acc1, ema_acc1)
            if run.is_main:
                left = (time.time() - began) * (args.epochs - epoch)
                logger.info("expected to finish at %s", (datetime.datetime.now() + datetime.timedelta(seconds=left)).strftime("%Y-%m-%d %H:%M:%S"))

    # ---------------------------------------------------------------- set-up, in the order main() needs it
    def _set_up(self, args):
        set_deterministic(args.seed, args.disable_uda)
        if args.workers > 0 and args.prefetch_factor < 1:
            raise ValueError(f"--prefetch-factor {args.prefetch_factor}: loader workers prefetch at least one batch each")
        if args.output_dir:
            utils.mkdir(args.output_dir)
        utils.init_distributed_mode(args)
        run = _Run(device=torch.device(args.device), is_main=utils.is_main_process())
        if run.is_main:
            logger.info("arguments: %s", args)
        train_set, test_set, run.train_sampler, test_sampler = self.load_data(args)
        classes = len(train_set.classes)
        shared = dict(batch_size=args.batch_size, num_workers=args.workers, pin_memory=not args.disable_pinmemory,
                      worker_init_fn=seed_worker, persistent_workers=args.persistent_workers and args.workers > 0,
                      prefetch_factor=args.prefetch_factor if args.workers > 0 else None)
        run.train_loader = torch.utils.data.DataLoader(train_set, sampler=run.train_sampler, collate_fn=_batch_mixer(args, classes), **shared)
        run.test_loader = torch.utils.data.DataLoader(test_set, sampler=test_sampler, **shared)

        run.bare_model = self.load_model(args, classes).to(run.device)
        if run.is_main:
            logger.info("model: %s", type(run.bare_model).__name__)
            logger.debug("%s", run.bare_model)
        if args.distributed and args.sync_bn:
            run.bare_model = nn.SyncBatchNorm.convert_sync_batchnorm(run.bare_model)
        run.criterion = nn.CrossEntropyLoss(label_smoothing=args.label_smoothing)
        run.optimizer = self.set_optimizer(args, _parameter_groups(run.bare_model, args.weight_decay, args.norm_weight_decay))
        fp16 = getattr(args, "amp_dtype", "bf16") == "fp16"
        run.scaler = torch.amp.GradScaler("cuda") if (fp16 and not args.disable_amp and run.device.type == "cuda") else None
        run.lr_scheduler = self.set_lr_scheduler(args, run.optimizer)
        if args.model_ema:
            # decay rescaled so that the averaging horizon (in samples) does not depend on world size, batch size,
            # update period or epoch count
            per_update = args.world_size * args.batch_size * args.model_ema_steps / args.epochs
            keep = 1.0 - min(1.0, (1.0 - args.model_ema_decay) * per_update)
            run.model_ema = utils.ExponentialMovingAverage(run.bare_model, device=run.device, decay=keep)

        name = self.get_tb_logdir_name(args)
        run.tb_dir, run.pt_dir = os.path.join(args.output_dir, name), os.path.join(args.output_dir, "pt", name)
        if args.print_logdir:
            if run.is_main:
                logger.info("TensorBoard directory: %s", run.tb_dir)
                logger.info("checkpoint directory: %s", run.pt_dir)
            return None
        if run.is_main:
            if args.clean:
                for folder in (run.tb_dir, run.pt_dir):
                    shutil.rmtree(folder, ignore_errors=True)
                logger.info("removed %s and %s", run.tb_dir, run.pt_dir)
            for folder in (run.tb_dir, run.pt_dir):
                os.makedirs(folder, exist_ok=args.resume is not None)      # a fresh run must not land in a used directory
        return run

    def _resume(self, args, run) -> None:
        path = os.path.join(run.pt_dir, "checkpoint_latest.pth") if args.resume == "latest" else args.resume
        saved = torch.load(path, map_location="cpu", weights_only=False)
        run.bare_model.load_state_dict(saved["model"])
        if not args.test_only:
            run.optimizer.load_state_dict(saved["optimizer"])
            if run.lr_scheduler is not None and saved.get("lr_scheduler") is not None:
                run.lr_scheduler.load_state_dict(saved["lr_scheduler"])
        args.start_epoch = saved["epoch"] + 1
        run.best = saved.get("max_test_acc1", -1.0)
        if run.model_ema:
            run.model_ema.load_state_dict(saved["model_ema"])
            run.best_ema = saved.get("max_ema_test_acc1", -1.0)
        if run.scaler and "scaler" in saved:
            run.scaler.load_state_dict(saved["scaler"])

    def _wrap_for_training(self, args, run) -> None:
        run.model = self.compile_model(args, run.bare_model)
        run.eval_model = self.get_eval_model(args, run.model, run.bare_model)
        if args.distributed:
            run.model = self._wrap_distributed(args, run.model, run.device)
            if hasattr(run.model, "guard_optimizer"):
                run.model.guard_optimizer(run.optimizer)
        if run.is_main:
            try:
                from torch.utils.tensorboard import SummaryWriter
                run.writer = SummaryWriter(run.tb_dir, purge_step=args.start_epoch)
            except Exception as problem:           # TensorBoard is optional
                logger.warning("no TensorBoard (%s): scalars go to the log only", problem)
            with open(os.path.join(run.tb_dir, "args.txt"), "w", encoding="utf-8") as f:
                f.write(f"{args}\n{' '.join(sys.argv)}")

    def _save_checkpoints(self, args, run, epoch: int, acc1: float, ema_acc1) -> None:
        """Rank 0 writes ``checkpoint_<epoch>.pth`` and ``checkpoint_latest.pth`` (plus the ``max_*`` files when a record
        fell) and drops the previous epoch's file; then ALL ranks meet at a barrier, so that nobody races ahead into the
        next epoch's collectives while rank 0 is still writing."""
        if run.is_main:
            record, run.best = acc1 > run.best, max(run.best, acc1)
            state = {"model": run.bare_model.state_dict(), "optimizer": run.optimizer.state_dict(),
                     "lr_scheduler": None if run.lr_scheduler is None else run.lr_scheduler.state_dict(), "epoch": epoch,
                     "args": args, "max_test_acc1": run.best}
            files = [f"checkpoint_{epoch}.pth", "checkpoint_latest.pth"] + (["checkpoint_max_test_acc1.pth"] if record else [])
            if run.model_ema:
                if ema_acc1 > run.best_ema:
                    files.append("checkpoint_max_ema_test_acc1.pth")
                run.best_ema = max(run.best_ema, ema_acc1)
                state.update(model_ema=run.model_ema.state_dict(), max_ema_test_acc1=run.best_ema)
            if run.scaler:
                state["scaler"] = run.scaler.state_dict()
            for name in files:
                utils.save_on_master(state, os.path.join(run.pt_dir, name))
            stale = os.path.join(run.pt_dir, f"checkpoint_{epoch - 1}.pth")
            if epoch > 0 and os.path.exists(stale):
                os.remove(stale)
        if utils.is_dist_avail_and_initialized():
            torch.distributed.barrier()

    # ------------------------------------------------------------- arguments
    def get_args_parser(self, add_help=True):
        """The command line of the reference trainer (same flags, destinations and defaults), built from :data:`ARGUMENTS`."""
        parser = argparse.ArgumentParser(description="Train an image classifier (spiking or not)", add_help=add_help)
        for flags, options in ARGUMENTS:
            parser.add_argument(*flags, **options)
        return parser


class _Run:
    """Everything one call of ``Trainer.main`` builds, in one place."""

    def __init__(self, device, is_main: bool):
        self.device, self.is_main = device, is_main
        self.train_loader = self.test_loader = self.train_sampler = None
        self.bare_model = self.model = self.eval_model = self.model_ema = None
        self.criterion = self.optimizer = self.lr_scheduler = self.scaler = None
        self.tb_dir = self.pt_dir = None
        self.writer = None
        self.best = self.best_ema = -1.0

    def log_scalars(self, epoch: int, **values) -> None:
        if self.writer is not None:
            for tag, value in values.items():
                self.writer.add_scalar(tag, value, epoch)


def _batch_mixer(args, num_classes: int):
    """Collate function applying mixup or cutmix (one of them, chosen per batch) when either is switched on."""
    if args.mixup_alpha <= 0.0 and args.cutmix_alpha <= 0.0:
        return None
    from torch.utils.data.dataloader import default_collate
    from .tv_ref_classify import transforms as T
    choices = []
    if args.mixup_alpha > 0.0:
        choices.append(T.RandomMixup(num_classes, p=1.0, alpha=args.mixup_alpha))
    if args.cutmix_alpha > 0.0:
        choices.append(T.RandomCutmix(num_classes, p=1.0, alpha=args.cutmix_alpha))
    return lambda batch: random.choice(choices)(*default_collate(batch))


_NORM_LAYERS = (nn.modules.batchnorm._BatchNorm, nn.LayerNorm, nn.GroupNorm, nn.modules.instancenorm._InstanceNorm, nn.LocalResponseNorm)


def _parameter_groups(model: nn.Module, weight_decay: float, norm_weight_decay):
    """All parameters, or two groups when normalisation layers get their own weight decay."""
    if norm_weight_decay is None:
        return model.parameters()
    norm, rest = [], []
    for module in model.modules():
        own = [p for p in module.parameters(recurse=False) if p.requires_grad]
        (norm if isinstance(module, _NORM_LAYERS) else rest).extend(own)
    groups = [{"params": rest, "weight_decay": weight_decay}, {"params": norm, "weight_decay": norm_weight_decay}]
    return [g for g in groups if g["params"]]


def _flag(*names, **options):
    return names, options


#: the command line: flag names, destinations and defaults are those of the reference trainer; the help text is ours
ARGUMENTS = (
    # data and model
    _flag("--data-path", default="/datasets01/imagenet_full_size/061417/", type=str, help="root folder of the dataset"),
    _flag("--model", default="resnet18", type=str, help="name handed to load_model()"),
    _flag("--device", default="cuda", type=str, help="cuda or cpu"),
    _flag("-b", "--batch-size", default=32, type=int, help="samples per process and step (global batch = processes x this)"),
    _flag("--epochs", default=90, type=int, metavar="N", help="passes over the training set"),
    _flag("-j", "--workers", default=16, type=int, metavar="N", help="loader worker processes"),
    _flag("--pretrained", dest="pretrained", action="store_true", help="start from the model zoo's weights"),
    _flag("--weights", default=None, type=str, help="name of a weights enum to load"),
    _flag("--prototype", dest="prototype", action="store_true", help="ignored (kept so that old command lines still parse)"),
    # optimisation
    _flag("--opt", default="sgd", type=str, help="sgd, sgd_nesterov, rmsprop or adamw"),
    _flag("--lr", default=0.1, type=float, help="peak learning rate"),
    _flag("--momentum", default=0.9, type=float, metavar="M", help="momentum of SGD / RMSprop"),
    _flag("--wd", "--weight-decay", default=0.0, type=float, metavar="W", dest="weight_decay", help="weight decay"),
    _flag("--norm-weight-decay", default=None, type=float, help="separate weight decay for normalisation layers (default: same as --wd)"),
    _flag("--label-smoothing", default=0.1, type=float, dest="label_smoothing", help="label smoothing of the cross entropy"),
    _flag("--mixup-alpha", default=0.2, type=float, help="mixup strength, 0 switches it off"),
    _flag("--cutmix-alpha", default=1.0, type=float, help="cutmix strength, 0 switches it off"),
    _flag("--clip-grad-norm", default=None, type=float, help="clip the global gradient norm to this value"),
    _flag("--lr-scheduler", default="cosa", type=str, help="step, cosa (cosine annealing) or exp"),
    _flag("--lr-warmup-epochs", default=5, type=int, help="epochs of warm-up before the main schedule, 0 for none"),
    _flag("--lr-warmup-method", default="linear", type=str, help="linear or constant"),
    _flag("--lr-warmup-decay", default=0.01, type=float, help="learning-rate factor at the start of the warm-up"),
    _flag("--lr-step-size", default=30, type=int, help="period of the step schedule in epochs"),
    _flag("--lr-gamma", default=0.1, type=float, help="factor of the step / exponential schedule"),
    _flag("--model-ema", action="store_true", help="keep an exponential moving average of the weights and evaluate it too"),
    _flag("--model-ema-steps", type=int, default=32, help="update the average every this many steps"),
    _flag("--model-ema-decay", type=float, default=0.99998, help="decay of the average, before rescaling to the run's size"),
    # augmentation and evaluation geometry
    _flag("--auto-augment", default="ta_wide", type=str, help="ra, ta_wide, augmix or an AutoAugment policy name"),
    _flag("--random-erase", default=0.1, type=float, help="probability of random erasing"),
    _flag("--interpolation", default="bilinear", type=str, help="resampling filter of the resizes"),
    _flag("--val-resize-size", default=232, type=int, help="shorter side after the validation resize"),
    _flag("--val-crop-size", default=224, type=int, help="centre crop used for validation"),
    _flag("--train-crop-size", default=176, type=int, help="random crop used for training"),
    _flag("--ra-sampler", action="store_true", help="repeated augmentation: every sample appears --ra-reps times per epoch, spread over the ranks"),
    _flag("--ra-reps", default=4, type=int, help="repetitions under --ra-sampler"),
    _flag("--cache-dataset", dest="cache_dataset", action="store_true", help="pickle the scanned image folders (with their transforms) for faster start-up"),
    # bookkeeping
    _flag("--output-dir", default="./logs", type=str, help="where logs and checkpoints go"),
    _flag("--resume", default=None, type=str, help="checkpoint to continue from; 'latest' picks checkpoint_latest.pth of this configuration"),
    _flag("--start-epoch", default=0, type=int, metavar="N", help="first epoch (set by --resume)"),
    _flag("--test-only", dest="test_only", action="store_true", help="evaluate and exit"),
    _flag("--seed", default=2020, type=int, help="seed of python, numpy and torch"),
    _flag("--print-logdir", action="store_true", help="print the log and checkpoint directories of this configuration and exit"),
    _flag("--clean", action="store_true", help="delete those directories first"),
    _flag("--disable-uda", action="store_true", help="do not call torch.use_deterministic_algorithms(True) (for operators without a deterministic kernel)"),
    # loader and precision
    _flag("--disable-pinmemory", action="store_true", help="unpinned host batches (less host memory, slower copies)"),
    _flag("--persistent-workers", action="store_true", help="keep loader workers between epochs"),
    _flag("--prefetch-factor", default=2, type=int, help="batches each worker keeps ready"),
    _flag("--disable-amp", action="store_true", help="full fp32 instead of autocast"),
    _flag("--amp-dtype", default="bf16", choices=("bf16", "fp16"), help="autocast dtype; only fp16 needs (and gets) a gradient scaler"),
    _flag("--compile", action="store_true", help="pass the model through torch.compile"),
    _flag("--compile-backend", default="inductor", type=str, help="torch.compile backend"),
    _flag("--compile-mode", default=None, type=str, help="torch.compile mode"),
    _flag("--compile-disable-cudagraphs", action="store_true", help="no CUDA graphs inside the inductor backend"),
    _flag("--compile-eval", action="store_true", help="evaluate the compiled model too (default: the eager one)"),
    # multi-process
    _flag("--sync-bn", dest="sync_bn", action="store_true", help="batch-norm statistics over all ranks"),
    _flag("--world-size", default=1, type=int, help="number of processes (filled in from the launcher's environment)"),
    _flag("--dist-url", default="env://", type=str, help="rendezvous URL"),
    _flag("--local_rank", type=int, help="set by old launchers; leave alone"),
)
