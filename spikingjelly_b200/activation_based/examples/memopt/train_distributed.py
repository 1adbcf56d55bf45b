"""One entry point for every distributed mode on the CIFAR10-DVS VGG: none | dp | tp | fsdp2 | fsdp2_tp | pp | auto
(role of ``examples/memopt/train_distributed.py`` in the reference).  Launch with torchrun for anything but ``none``:

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m spikingjelly_b200.activation_based.examples.memopt.train_distributed --distributed-mode dp --synthetic --max-steps 5

``--prefer speed|memory|capacity`` asks the planner; with ``--distributed-mode auto`` its whole recommendation is applied.
``--memopt-level`` runs the automatic memory optimisation (spike compression + checkpointing) before parallelisation.
"""
import argparse
import os
import time

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ... import distributed as D
from ... import functional
from ...memopt import memory_optimization
from .models import CIFAR10DVSVGG, VGGBlock


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="Distributed SNN training example for CIFAR10-DVS.")
    p.add_argument("--data-dir", type=str, default=None)
    p.add_argument("--synthetic", action="store_true")
    p.add_argument("--epochs", type=int, default=1)
    p.add_argument("--max-steps", type=int, default=0)
    p.add_argument("--batch-size", type=int, default=16)
    p.add_argument("--lr", type=float, default=1e-3)
    p.add_argument("--weight-decay", type=float, default=0.0)
    p.add_argument("--T", type=int, default=10)
    p.add_argument("--resolution", type=int, default=48)
    p.add_argument("--backend", type=str, default="auto")
    p.add_argument("--distributed-mode", default="none", choices=("auto", "none", "dp", "tp", "fsdp2", "fsdp2_tp", "pp"))
    p.add_argument("--prefer", default=None, choices=D.SNN_DISTRIBUTED_PREFERENCES)
    p.add_argument("--mesh-shape", type=int, nargs="*", default=None)
    p.add_argument("--tp-mesh-dim", type=int, default=0)
    p.add_argument("--dp-mesh-dim", type=int, default=None)
    p.add_argument("--optimizer-sharding", default=None, choices=("none", "zero"))
    p.add_argument("--memopt-level", type=int, default=None)
    p.add_argument("--memopt-compress-x", action="store_true")
    p.add_argument("--print-summary", action="store_true")
    return p.parse_args(argv)


def setup_runtime(args):
    launched = "RANK" in os.environ and "WORLD_SIZE" in os.environ
    if args.distributed_mode == "none" or (args.distributed_mode == "auto" and not launched):
        args.distributed_mode = "none"
        return 0, 1, torch.device("cuda" if torch.cuda.is_available() else "cpu")
    if not launched:
        raise RuntimeError(f"distributed_mode='{args.distributed_mode}' requires torchrun (RANK / WORLD_SIZE / LOCAL_RANK).")
    local = int(os.environ.get("LOCAL_RANK", 0))
    device = torch.device("cuda", local) if torch.cuda.is_available() else torch.device("cpu")
    if device.type == "cuda":
        torch.cuda.set_device(local)
    D.ensure_distributed_initialized()
    return dist.get_rank(), dist.get_world_size(), device


def synthetic_loader(args, device, rank):
    g = torch.Generator().manual_seed(1234 + rank)
    n = args.batch_size * max(args.max_steps, 4)
    y = torch.randint(0, 10, (n,), generator=g)
    x = (torch.rand(n, args.T, 2, args.resolution, args.resolution, generator=g) < (0.05 + 0.01 * y.view(-1, 1, 1, 1, 1))).float()
    return torch.utils.data.DataLoader(torch.utils.data.TensorDataset(x, y), batch_size=args.batch_size, drop_last=True)


def real_loader(args, rank, world):
    from ....datasets.cifar10_dvs import CIFAR10DVS
    from ....datasets.utils import fast_split_to_train_test_set
    full = CIFAR10DVS(args.data_dir, data_type="frame", frames_number=args.T, split_by="number")
    train, _ = fast_split_to_train_test_set(0.9, full, 10)
    sampler = torch.utils.data.distributed.DistributedSampler(train, world, rank) if world > 1 else None
    return torch.utils.data.DataLoader(train, batch_size=args.batch_size, sampler=sampler, shuffle=sampler is None, drop_last=True,
                                       num_workers=4, pin_memory=True)


def main(argv=None):
    args = parse_args(argv)
    rank, world, device = setup_runtime(args)
    backend = ("cuda" if device.type == "cuda" else "torch") if args.backend == "auto" else args.backend
    if args.prefer is not None:
        rec = D.recommend_snn_distributed_strategy(model="cifar10dvs_vgg", world_size=world, prefer=args.prefer,
                                                   batch_size=args.batch_size, backend=backend)
        if args.distributed_mode == "auto":
            args.distributed_mode, args.optimizer_sharding, args.memopt_level = rec.mode, rec.optimizer_sharding, rec.memopt_level
            if args.mesh_shape is None and rec.mesh_shape is not None:
                args.mesh_shape = list(rec.mesh_shape)
        elif args.memopt_level is None:
            args.memopt_level = rec.memopt_level
        if rank == 0:
            print(f"planner: mode={rec.mode} optimizer_sharding={rec.optimizer_sharding} memopt_level={rec.memopt_level}")
    elif args.distributed_mode == "auto":
        raise ValueError("--distributed-mode auto requires --prefer speed|memory|capacity.")

    net = CIFAR10DVSVGG(backend=backend, resolution=args.resolution).to(device)
    if args.memopt_level:
        dummy = torch.zeros(args.batch_size, args.T, 2, args.resolution, args.resolution, device=device)
        net = memory_optimization(net, (VGGBlock,), dummy_input=(dummy,), compress_x=args.memopt_compress_x, level=args.memopt_level,
                                  verbose=args.print_summary and rank == 0)
    optimizer = None
    if args.distributed_mode != "none":
        cfg = D.SNNDistributedConfig(mode=args.distributed_mode, device_type=device.type,
                                     mesh_shape=tuple(args.mesh_shape) if args.mesh_shape else None, tp_mesh_dim=args.tp_mesh_dim,
                                     dp_mesh_dim=args.dp_mesh_dim, tensor_parallel_roots=("classifier",), conv_tensor_parallel_roots=("features",))
        net, mesh, analysis = D.configure_snn_distributed(net, cfg)
        if args.print_summary and rank == 0:
            print(analysis)
        optimizer = D.build_snn_optimizer(net, args.distributed_mode, lr=args.lr, weight_decay=args.weight_decay, optimizer_sharding=args.optimizer_sharding or "none")
    if optimizer is None:
        optimizer = torch.optim.AdamW(net.parameters(), lr=args.lr, weight_decay=args.weight_decay)
    if hasattr(net, "guard_optimizer"):
        net.guard_optimizer(optimizer)

    loader = synthetic_loader(args, device, rank) if args.synthetic or args.data_dir is None else real_loader(args, rank, world)
    for epoch in range(args.epochs):
        net.train()
        seen, t0, loss_sum = 0, time.time(), 0.0
        for step, (x, y) in enumerate(loader):
            if args.max_steps and step >= args.max_steps:
                break
            x, y = x.to(device, non_blocking=True), y.to(device, non_blocking=True)
            out = D.materialize_dtensor_output(net(x)) if hasattr(D, "materialize_dtensor_output") else net(x)
            loss = F.cross_entropy(out.mean(0), y)
            optimizer.zero_grad(set_to_none=True)
            loss.backward()
            optimizer.step()
            functional.reset_net(net)
            seen += y.numel()
            loss_sum += loss.item()
        if device.type == "cuda":
            torch.cuda.synchronize()
        if hasattr(net, "check_communication"):
            net.check_communication()        # raises CommError if a gradient exchange of this epoch gave up on a peer
        if rank == 0:
            print(f"epoch {epoch}: mean loss {loss_sum / max(step, 1):.4f}, {seen * world / (time.time() - t0):.1f} samples/s over {world} rank(s), "
                  f"mode {args.distributed_mode}")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
