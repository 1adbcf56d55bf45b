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
        set_deterministic(args.seed, args.disable_uda)
        if args.workers > 0 and args.prefetch_factor < 1:
            raise ValueError(f"--prefetch-factor must be >= 1 when --workers > 0, but got {args.prefetch_factor}.")
        if args.output_dir:
            utils.mkdir(args.output_dir)
        utils.init_distributed_mode(args)
        main_proc = utils.is_main_process()
        if main_proc:
            logger.info("Training arguments: %s", args)
        device = torch.device(args.device)

        dataset, dataset_test, train_sampler, test_sampler = self.load_data(args)
        num_classes = len(dataset.classes)
        collate_fn = None
        mixers = []
        if args.mixup_alpha > 0.0 or args.cutmix_alpha > 0.0:
            from torch.utils.data.dataloader import default_collate
            from .tv_ref_classify import transforms as T
            if args.mixup_alpha > 0.0:
                mixers.append(T.RandomMixup(num_classes, p=1.0, alpha=args.mixup_alpha))
            if args.cutmix_alpha > 0.0:
                mixers.append(T.RandomCutmix(num_classes, p=1.0, alpha=args.cutmix_alpha))

            def collate_fn(batch):
                return random.choice(mixers)(*default_collate(batch))
        loader_kw = dict(batch_size=args.batch_size, num_workers=args.workers, pin_memory=not args.disable_pinmemory,
                         worker_init_fn=seed_worker, persistent_workers=args.persistent_workers and args.workers > 0,
                         prefetch_factor=(args.prefetch_factor if args.workers > 0 else None))
        data_loader = torch.utils.data.DataLoader(dataset, sampler=train_sampler, collate_fn=collate_fn, **loader_kw)
        data_loader_test = torch.utils.data.DataLoader(dataset_test, sampler=test_sampler, **loader_kw)

        model = self.load_model(args, num_classes)
        model.to(device)
        if main_proc:
            logger.info("Model created: %s", type(model).__name__)
            logger.debug("Model architecture:\n%s", model)
        if args.distributed and args.sync_bn:
            model = torch.nn.SyncBatchNorm.convert_sync_batchnorm(model)
        criterion = nn.CrossEntropyLoss(label_smoothing=args.label_smoothing)

        if args.norm_weight_decay is None:
            parameters = model.parameters()
        else:
            norm_classes = (nn.modules.batchnorm._BatchNorm, nn.LayerNorm, nn.GroupNorm, nn.modules.instancenorm._InstanceNorm,
                            nn.LocalResponseNorm)
            norm_params, other_params = [], []
            for m in model.modules():
                bucket = norm_params if isinstance(m, norm_classes) else other_params
                bucket.extend(p for p in m.parameters(recurse=False) if p.requires_grad)
            parameters = [{"params": p, "weight_decay": w} for p, w in
                          ((norm_params, args.norm_weight_decay), (other_params, args.weight_decay)) if p]
        optimizer = self.set_optimizer(args, parameters)
        use_scaler = (not args.disable_amp) and device.type == "cuda" and getattr(args, "amp_dtype", "bf16") == "fp16"
        scaler = torch.amp.GradScaler("cuda") if use_scaler else None
        lr_scheduler = self.set_lr_scheduler(args, optimizer)
        model_without_ddp = model

        model_ema = None
        if args.model_ema:
            # keep the EMA horizon independent of world size, batch size, update period and epoch count
            adjust = args.world_size * args.batch_size * args.model_ema_steps / args.epochs
            alpha = min(1.0, (1.0 - args.model_ema_decay) * adjust)
            model_ema = utils.ExponentialMovingAverage(model_without_ddp, device=device, decay=1.0 - alpha)

        tb_name = self.get_tb_logdir_name(args)
        pt_dir = os.path.join(args.output_dir, "pt", tb_name)
        tb_dir = os.path.join(args.output_dir, tb_name)
        if args.print_logdir:
            if main_proc:
                logger.info("TensorBoard log directory: %s", tb_dir)
                logger.info("Checkpoint directory: %s", pt_dir)
            sys.exit()
        if args.clean and main_proc:
            for d in (tb_dir, pt_dir):
                if os.path.exists(d):
                    shutil.rmtree(d)
            logger.info("remove %s and %s.", tb_dir, pt_dir)
        if main_proc:
            os.makedirs(tb_dir, exist_ok=args.resume is not None)
            os.makedirs(pt_dir, exist_ok=args.resume is not None)

        max_test_acc1, max_ema_test_acc1 = -1.0, -1.0
        if args.resume is not None:
            path = os.path.join(pt_dir, "checkpoint_latest.pth") if args.resume == "latest" else args.resume
            checkpoint = torch.load(path, map_location="cpu", weights_only=False)
            model_without_ddp.load_state_dict(checkpoint["model"])
            if not args.test_only:
                optimizer.load_state_dict(checkpoint["optimizer"])
                lr_scheduler.load_state_dict(checkpoint["lr_scheduler"])
            args.start_epoch = checkpoint["epoch"] + 1
            if model_ema:
                model_ema.load_state_dict(checkpoint["model_ema"])
                max_ema_test_acc1 = checkpoint.get("max_ema_test_acc1", -1.0)
            if scaler and "scaler" in checkpoint:
                scaler.load_state_dict(checkpoint["scaler"])
            max_test_acc1 = checkpoint.get("max_test_acc1", -1.0)

        model = self.compile_model(args, model_without_ddp)
        eval_model = self.get_eval_model(args, model, model_without_ddp)
        if args.distributed:
            model = self._wrap_distributed(args, model, device)

        tb_writer = None
        if main_proc:
            try:
                from torch.utils.tensorboard import SummaryWriter
                tb_writer = SummaryWriter(tb_dir, purge_step=args.start_epoch)
            except Exception as e:                 # TensorBoard is optional
                logger.warning("TensorBoard unavailable (%s); scalars are only logged.", e)
            with open(os.path.join(tb_dir, "args.txt"), "w", encoding="utf-8") as f:
                f.write(str(args) + "\n" + " ".join(sys.argv))

        def scalars(epoch, **kv):
            if tb_writer is not None:
                for k, v in kv.items():
                    tb_writer.add_scalar(k, v, epoch)

        if args.test_only:
            if model_ema:
                self.evaluate(args, model_ema, criterion, data_loader_test, device=device, log_suffix="EMA")
            else:
                self.evaluate(args, eval_model, criterion, data_loader_test, device=device)
            return

        for epoch in range(args.start_epoch, args.epochs):
            t0 = time.time()
            if args.distributed:
                train_sampler.set_epoch(epoch)
            self.before_train_one_epoch(args, model, epoch)
            train_loss, train_acc1, train_acc5 = self.train_one_epoch(model, criterion, optimizer, data_loader, device, epoch,
                                                                      args, model_ema, scaler)
            scalars(epoch, train_loss=train_loss, train_acc1=train_acc1, train_acc5=train_acc5)
            if lr_scheduler is not None:
                lr_scheduler.step()
            self.before_test_one_epoch(args, eval_model, epoch)
            test_loss, test_acc1, test_acc5 = self.evaluate(args, eval_model, criterion, data_loader_test, device=device)
            scalars(epoch, test_loss=test_loss, test_acc1=test_acc1, test_acc5=test_acc5)
            if model_ema:
                ema_loss, ema_acc1, ema_acc5 = self.evaluate(args, model_ema, criterion, data_loader_test, device=device,
                                                             log_suffix="EMA")
                scalars(epoch, ema_test_loss=ema_loss, ema_test_acc1=ema_acc1, ema_test_acc5=ema_acc5)
            if main_proc:
                is_best = test_acc1 > max_test_acc1
                max_test_acc1 = max(max_test_acc1, test_acc1)
                checkpoint = {"model": model_without_ddp.state_dict(), "optimizer": optimizer.state_dict(),
                              "lr_scheduler": lr_scheduler.state_dict() if lr_scheduler is not None else None,
                              "epoch": epoch, "args": args, "max_test_acc1": max_test_acc1}
                is_best_ema = False
                if model_ema:
                    is_best_ema = ema_acc1 > max_ema_test_acc1
                    max_ema_test_acc1 = max(max_ema_test_acc1, ema_acc1)
                    checkpoint["model_ema"] = model_ema.state_dict()
                    checkpoint["max_ema_test_acc1"] = max_ema_test_acc1
                if scaler:
                    checkpoint["scaler"] = scaler.state_dict()
                names = [f"checkpoint_{epoch}.pth", "checkpoint_latest.pth"]
                names += ["checkpoint_max_test_acc1.pth"] if is_best else []
                names += ["checkpoint_max_ema_test_acc1.pth"] if is_best_ema else []
                for name in names:
                    utils.save_on_master(checkpoint, os.path.join(pt_dir, name))
                previous = os.path.join(pt_dir, f"checkpoint_{epoch - 1}.pth")
                if epoch > 0 and os.path.exists(previous):
                    os.remove(previous)
                eta = datetime.datetime.now() + datetime.timedelta(seconds=(time.time() - t0) * (args.epochs - epoch))
                logger.info("Estimated finish time: %s", eta.strftime("%Y-%m-%d %H:%M:%S"))

    # ------------------------------------------------------------- arguments
    def get_args_parser(self, add_help=True):
        p = argparse.ArgumentParser(description="PyTorch Classification Training", add_help=add_help)
        a = p.add_argument
        a("--data-path", default="/datasets01/imagenet_full_size/061417/", type=str, help="dataset path")
        a("--model", default="resnet18", type=str, help="model name")
        a("--device", default="cuda", type=str, help="device (Use cuda or cpu Default: cuda)")
        a("-b", "--batch-size", default=32, type=int, help="images per gpu, the total batch size is $NGPU x batch_size")
        a("--epochs", default=90, type=int, metavar="N", help="number of total epochs to run")
        a("-j", "--workers", default=16, type=int, metavar="N", help="number of data loading workers (default: 16)")
        a("--opt", default="sgd", type=str, help="optimizer")
        a("--lr", default=0.1, type=float, help="initial learning rate")
        a("--momentum", default=0.9, type=float, metavar="M", help="momentum")
        a("--wd", "--weight-decay", default=0.0, type=float, metavar="W", help="weight decay (default: 0.)", dest="weight_decay")
        a("--norm-weight-decay", default=None, type=float, help="weight decay for Normalization layers (default: None, same value as --wd)")
        a("--label-smoothing", default=0.1, type=float, help="label smoothing (default: 0.1)", dest="label_smoothing")
        a("--mixup-alpha", default=0.2, type=float, help="mixup alpha (default: 0.2)")
        a("--cutmix-alpha", default=1.0, type=float, help="cutmix alpha (default: 1.0)")
        a("--lr-scheduler", default="cosa", type=str, help="the lr scheduler (default: cosa)")
        a("--lr-warmup-epochs", default=5, type=int, help="the number of epochs to warmup (default: 5)")
        a("--lr-warmup-method", default="linear", type=str, help="the warmup method (default: linear)")
        a("--lr-warmup-decay", default=0.01, type=float, help="the decay for lr")
        a("--lr-step-size", default=30, type=int, help="decrease lr every step-size epochs")
        a("--lr-gamma", default=0.1, type=float, help="decrease lr by a factor of lr-gamma")
        a("--output-dir", default="./logs", type=str, help="path to save outputs")
        a("--resume", default=None, type=str, help="path of checkpoint. If set to 'latest', it will try to load the latest checkpoint")
        a("--start-epoch", default=0, type=int, metavar="N", help="start epoch")
        a("--cache-dataset", dest="cache_dataset", action="store_true", help="Cache the datasets for quicker initialization. It also serializes the transforms")
        a("--sync-bn", dest="sync_bn", action="store_true", help="Use sync batch norm")
        a("--test-only", dest="test_only", action="store_true", help="Only test the model")
        a("--pretrained", dest="pretrained", action="store_true", help="Use pre-trained models from the modelzoo")
        a("--auto-augment", default="ta_wide", type=str, help="auto augment policy (default: ta_wide)")
        a("--random-erase", default=0.1, type=float, help="random erasing probability (default: 0.1)")
        a("--world-size", default=1, type=int, help="number of distributed processes")
        a("--dist-url", default="env://", type=str, help="url used to set up distributed training")
        a("--model-ema", action="store_true", help="enable tracking Exponential Moving Average of model parameters")
        a("--model-ema-steps", type=int, default=32, help="the number of iterations that controls how often to update the EMA model (default: 32)")
        a("--model-ema-decay", type=float, default=0.99998, help="decay factor for Exponential Moving Average of model parameters (default: 0.99998)")
        a("--interpolation", default="bilinear", type=str, help="the interpolation method (default: bilinear)")
        a("--val-resize-size", default=232, type=int, help="the resize size used for validation (default: 232)")
        a("--val-crop-size", default=224, type=int, help="the central crop size used for validation (default: 224)")
        a("--train-crop-size", default=176, type=int, help="the random crop size used for training (default: 176)")
        a("--clip-grad-norm", default=None, type=float, help="the maximum gradient norm (default None)")
        a("--ra-sampler", action="store_true", help="whether to use Repeated Augmentation in training")
        a("--ra-reps", default=4, type=int, help="number of repetitions for Repeated Augmentation (default: 4)")
        a("--prototype", dest="prototype", action="store_true", help="accepted for compatibility; torchvision's prototype API no longer exists")
        a("--weights", default=None, type=str, help="the weights enum name to load")
        a("--seed", default=2020, type=int, help="the random seed")
        a("--print-logdir", action="store_true", help="print the dirs for tensorboard logs and pt files and exit")
        a("--clean", action="store_true", help="delete the dirs for tensorboard logs and pt files")
        a("--disable-pinmemory", action="store_true", help="not use pin memory in dataloader, which can help reduce memory consumption")
        a("--persistent-workers", action="store_true", help="keep DataLoader workers alive across epochs")
        a("--prefetch-factor", default=2, type=int, help="number of batches loaded in advance by each worker")
        a("--disable-amp", action="store_true", help="not use automatic mixed precision training")
        a("--amp-dtype", default="bf16", choices=("bf16", "fp16"), help="autocast dtype (bf16 needs no gradient scaler)")
        a("--compile", action="store_true", help="wrap the model with torch.compile")
        a("--compile-backend", default="inductor", type=str, help="torch.compile backend")
        a("--compile-mode", default=None, type=str, help="torch.compile mode")
        a("--compile-disable-cudagraphs", action="store_true", help="disable CUDA graphs inside the inductor backend")
        a("--compile-eval", action="store_true", help="also evaluate with the compiled model")
        a("--local_rank", type=int, help="args for DDP, which should not be set by user")
        a("--disable-uda", action="store_true", help="not set 'torch.use_deterministic_algorithms(True)', which can avoid the error raised by some functions that do not have a deterministic implementation")
        return p
