#!/usr/bin/env python
"""Flagship benchmark: Spikformer-8-512 training throughput (samples/s), data parallel.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 20 --warmup 5
    python bench.py --impl reference ...      # the unmodified reference from baseline/_ref
    python bench.py --config sew_resnet|snn_llm|neuron ...   # the other benchmark configurations, same JSON contract

Workload (identical for both arms): Spikformer with 8 encoder blocks, d=512, 8 heads, MLP
ratio 4, T=4, 224x224x3 synthetic N(0,1) images, 1000 random classes, per-GPU batch 32 (global
256 at 8 GPUs, weak scaling), bf16 autocast, cross entropy on the rate over T, AdamW step,
``reset_net`` — all inside the timed region.  Weights are random-init.

Timing: W warm-up steps, then K steps between CUDA events with a barrier + synchronize on
both sides; the reported time is the max over ranks.  L2 is flushed (256 MB write) between
steps.  ``value`` uses device-resident inputs; ``e2e`` adds, per step, the pinned-host to
device copy of the batch and a device-to-host read of the loss.
Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent

MODEL_CFG = dict(T=4, in_channels=3, img_size_h=224, img_size_w=224, num_classes=1000, embed_dims=512,
                 num_heads=8, mlp_ratio=4.0, depths=8)
PER_GPU_BATCH = 32


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", choices=["ours", "reference"], default="ours")
    p.add_argument("--batch", type=int, default=PER_GPU_BATCH, help="per-GPU batch")
    p.add_argument("--ref-backend", default="auto", help="reference neuron backend: auto|triton|torch")
    p.add_argument("--ref-compile", action="store_true",
                   help="reference arm: wrap the model in torch.compile (the reference's stock modules are compile-friendly; its "
                        "\"inductor\" backend name exists for FlexSN only, LIFNode offers torch / cupy / triton)")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--config", choices=["spikformer", "sew_resnet", "snn_llm", "neuron"], default="spikformer",
                   help="spikformer (default, the headline): Spikformer-8-512 data parallel; sew_resnet: SEW-ResNet-18 on event frames, "
                        "data parallel; snn_llm: the 24-layer spike-driven LM, tensor parallel; neuron: multi-step LIF forward + backward")
    p.add_argument("--batch-default", action="store_true", help=argparse.SUPPRESS)
    return p.parse_args()


class ClockSampler:
    """Samples SM clocks / throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [s.strip() for s in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


class _Prefetcher:
    """Side-stream copies of the next batch (the same logic as ``spikingjelly_b200.utils.prefetch.DevicePrefetcher``, kept
    here so that the reference arm imports nothing of this package)."""

    def __init__(self, torch, device):
        self.torch, self.device, self.stream = torch, device, torch.cuda.Stream(device)

    def stage(self, *host):
        torch = self.torch
        with torch.cuda.stream(self.stream):
            out = tuple(t.to(self.device, non_blocking=True) for t in host)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        return out, ev

    def take(self, staged):
        out, ev = staged
        cur = self.torch.cuda.current_stream(self.device)
        cur.wait_event(ev)
        for t in out:
            t.record_stream(cur)
        return out


class _Deferred:
    """Non-blocking read-back of a device scalar; ``get()`` waits for the copy."""

    _ring, _next = [], 0          # four pinned scalars, reused in turn: at most two reads are in flight at a time

    def __init__(self, torch, value):
        v = value.detach().reshape(1)
        cls = type(self)
        if len(cls._ring) < 4:
            cls._ring.append(torch.empty(1, dtype=torch.float32, pin_memory=True))
        self.host = cls._ring[cls._next % len(cls._ring)]
        cls._next += 1
        self.host.copy_(v.float(), non_blocking=True)
        self.event = torch.cuda.Event()
        self.event.record(torch.cuda.current_stream(v.device))

    def get(self) -> float:
        self.event.synchronize()
        return float(self.host.item())


# Workloads that share the data-parallel training loop below.  ``x``: shape of one per-GPU batch, ``classes``, how the
# synthetic input is drawn, and how each arm builds the network.
def _sew_build(impl, device, ref_backend):
    sys.path.insert(0, str(ROOT))
    from benchmark.benchmark_sew_resnet import build
    net, functional = build(impl, device)
    return net, functional, ("triton" if impl == "reference" else None)


WORKLOADS = {
    "spikformer": dict(
        model="Spikformer-8-512", T=4, batch=PER_GPU_BATCH, classes=1000, seq_len=196,
        shape=lambda B: (B, 3, 224, 224), draw=lambda torch, shape, device: torch.randn(*shape, device=device),
        metric="train samples/sec (Spikformer-8-512, T=4, bf16, data parallel, device-timed, max over ranks)",
        data="synthetic N(0,1) 224x224x3 images, random labels, random-init weights"),
    "sew_resnet": dict(
        model="SEW-ResNet-18 (ADD, LIF tau 2, ATan)", T=16, batch=32, classes=11, seq_len=None,
        shape=lambda B: (16, B, 2, 128, 128),
        draw=lambda torch, shape, device: (torch.poisson(torch.full(shape, 0.05, device=device)) > 0).float(),
        metric="train samples/sec (SEW-ResNet-18, T=16, 2x128x128 event frames, bf16, data parallel, device-timed, max over ranks)",
        data="synthetic Poisson(0.05) event frames clipped to {0,1}, random labels over 11 classes, random-init weights"),
}


def build_ours(device, backend="cuda"):
    from spikingjelly_b200 import ops
    from spikingjelly_b200.activation_based import functional
    from spikingjelly_b200.models import spikformer
    ops.require()
    net = spikformer.Spikformer(backend=backend, **MODEL_CFG).to(device)
    return net, functional


def build_reference(device, backend):
    ref_dir = ROOT / "baseline" / "_ref"
    if not (ref_dir / "spikingjelly").exists():
        raise FileNotFoundError("baseline/_ref is empty: the reference is not installed")
    sys.path.insert(0, str(ref_dir))
    from spikingjelly.activation_based import functional
    from spikingjelly.activation_based.model import spikformer
    chosen = backend
    if backend == "auto":
        chosen = "triton"
        try:
            import torch
            from spikingjelly.activation_based import neuron
            probe = neuron.LIFNode(step_mode="m", backend="triton").to(device)
            x = torch.randn(4, 1024, device=device, dtype=torch.bfloat16, requires_grad=True)
            probe(x).sum().backward()
            torch.cuda.synchronize()
        except Exception as exc:  # Triton path unusable here: the eager backend is the stock fallback
            sys.stderr.write(f"[bench] reference triton backend unavailable ({type(exc).__name__}: {exc}); using torch\n")
            chosen = "torch"
    net = spikformer.Spikformer(backend=chosen, **MODEL_CFG).to(device)
    return net, functional, chosen


def run_delegated(args) -> None:
    """``--config snn_llm`` / ``--config neuron``: run the configuration's own benchmark (same process, same launcher) and
    restate its record in this script's JSON contract."""
    import contextlib
    import io
    import runpy
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    if rank == 0:
        sampler.start()
    buf = io.StringIO()
    if args.config == "snn_llm":
        argv = ["benchmark_snn_llm.py", "--steps", str(args.steps), "--warmup", str(args.warmup), "--impl", args.impl]
        if args.impl == "ours" and world > 1:
            argv += ["--path", "fused"]
        script = ROOT / "benchmark" / "benchmark_snn_llm.py"
    else:
        argv = ["benchmark_neuron_kernels.py", "--headline", "--iters", str(max(args.steps, 5)), "--impl", args.impl]
        script = ROOT / "benchmark" / "benchmark_neuron_kernels.py"
    old_argv = sys.argv
    sys.argv = argv
    try:
        with contextlib.redirect_stdout(buf):
            runpy.run_path(str(script), run_name="__main__")
    finally:
        sys.argv = old_argv
    clocks = sampler.stop() if rank == 0 else {}
    if rank != 0:
        return
    lines = [ln for ln in buf.getvalue().splitlines() if ln.startswith("{")]
    src = json.loads(lines[-1]) if lines else {"unavailable": "the benchmark printed no record"}
    if "unavailable" in src:
        print(json.dumps({"impl": args.impl, "unavailable": src["unavailable"]}))
        return
    if args.config == "snn_llm":
        rec = {"metric": "train tokens/sec (SNN-LLM 24L d2048 FFN5504 T=4, seq 2048, micro-batch 4, tensor parallel, device-timed, max over ranks)",
               "value": src["tokens_per_s"], "unit": "tokens/s", "ms_per_step": src["ms_per_step"], "higher_is_better": True,
               "scaling": "strong", "config": {"model": "SNN-LLM-24L-2048", "T": 4, "global_batch": 4, "seq_len": 2048,
                                               "parallelism": f"tp{world}", "path": src.get("path"), "l2": "256 MB flush written between steps"}}
    else:
        rec = {"metric": "multi-step LIF forward+backward, T=4, N=2^24, bf16 (us, CUDA events, L2 flushed)", "value": src["fwd_bwd_us"],
               "unit": "us", "ms_per_step": round(src["fwd_bwd_us"] / 1e3, 4), "higher_is_better": False, "scaling": "weak",
               "config": {"model": "LIFNode tau=2 hard reset ATan", "T": 4, "N": 1 << 24, "seq_len": None, "global_batch": None,
                          "parallelism": "1 GPU", "l2": "256 MB flush written between launches"}}
    rec.update({"n_gpus": world, "steps": args.steps, "warmup": args.warmup, "vs_baseline": None, "dtype": "bf16",
                "data": "synthetic", "impl": args.impl, "clocks": clocks, "source_record": src})
    print(json.dumps(rec))


def main():
    args = parse()
    if args.config in ("snn_llm", "neuron"):
        return run_delegated(args)
    wl = WORKLOADS[args.config]
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "no CUDA device in this process"}))
            return
        raise SystemExit("bench.py needs a CUDA device")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    if args.gpus != world and rank == 0:
        sys.stderr.write(f"[bench] --gpus {args.gpus} but WORLD_SIZE={world}; using WORLD_SIZE\n")

    torch.manual_seed(1234 + rank)
    torch.backends.cudnn.benchmark = True
    extra = {}
    launches = None
    if args.impl == "reference":
        try:
            if args.config == "spikformer":
                net, functional, chosen = build_reference(device, args.ref_backend)
            else:
                net, functional, chosen = _sew_build("reference", device, args.ref_backend)
        except Exception as exc:
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": f"{type(exc).__name__}: {exc}"[:300]}))
            return
        extra["reference_backend"] = chosen
        if args.ref_compile:
            net = torch.compile(net)
            extra["reference_compiled"] = True
        if world > 1:
            from spikingjelly.activation_based.distributed.data_parallel import prepare_snn_data_parallel
            net = prepare_snn_data_parallel(net, device_ids=[local_rank])
        step_model = net
    else:
        if args.config == "spikformer":
            net, functional = build_ours(device)
        else:
            net, functional, _ = _sew_build("ours", device, None)
        if world > 1:
            from spikingjelly_b200.parallel import data_parallel
            step_model = data_parallel.prepare_snn_data_parallel(net, device_ids=[local_rank])
        else:
            step_model = net
        from spikingjelly_b200.ops import counters
        launches = counters

    opt = torch.optim.AdamW(step_model.parameters(), lr=1e-4, weight_decay=0.01, fused=True)
    B = args.batch if args.batch != PER_GPU_BATCH or args.config == "spikformer" else wl["batch"]
    shape = wl["shape"](B)
    dev_x = wl["draw"](torch, shape, device)
    dev_y = torch.randint(0, wl["classes"], (B,), device=device)
    host_x = [wl["draw"](torch, shape, "cpu").pin_memory() for _ in range(2)]
    host_y = [torch.randint(0, wl["classes"], (B,)).pin_memory() for _ in range(2)]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)

    def train_step(x, y):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            out = step_model(x)
        loss = F.cross_entropy(out.float().mean(0), y)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        functional.reset_net(net)
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def check_comm():
        # a gradient exchange whose peer wait ran out raises here: its throughput must not be reported
        check = getattr(step_model, "check_communication", None)
        if check is not None:
            check()

    for _ in range(args.warmup):
        train_step(dev_x, dev_y)
        flush.zero_()
    barrier()

    # ---- device-resident timing ------------------------------------------------
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    if launches is not None:
        launches.reset()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(args.steps):
        loss = train_step(dev_x, dev_y)
        flush.zero_()
    ev1.record()
    barrier()
    check_comm()
    ms = ev0.elapsed_time(ev1)
    n_launch = launches.total() if launches is not None else None
    t = torch.tensor([ms], device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())
    clocks = sampler.stop() if rank == 0 else {}

    # ---- end-to-end timing: pinned host -> device every step, loss read back ----
    e2e = None
    if not args.no_e2e:
        # The loop a user writes with utils.prefetch: the NEXT batch is copied from pinned memory on a side stream while
        # this step computes, and the loss of step i is read on the host after step i + 1 has been launched (its copy is
        # queued right behind step i).  Every step still pays one H2D copy of its inputs and one D2H read of its loss
        # inside the timed region; both arms run the same loop.
        pf = _Prefetcher(torch, device)

        def pipelined(n):
            staged = pf.stage(host_x[0], host_y[0])
            pending = value = None
            for i in range(n):
                x, y = pf.take(staged)
                if i + 1 < n:
                    staged = pf.stage(host_x[(i + 1) % 2], host_y[(i + 1) % 2])
                reader = _Deferred(torch, train_step(x, y))
                if pending is not None:
                    value = pending.get()
                pending = reader
                flush.zero_()
            return pending.get() if pending is not None else value
        # warm-up through the same loop: the side stream's memory pool and the pinned read-back buffers are allocated here,
        # not inside the timed region (a first pinned allocation costs milliseconds)
        pipelined(max(3, min(args.warmup, 5)))
        barrier()
        t0 = time.perf_counter()
        ev0.record()
        loss_val = pipelined(args.steps)
        ev1.record()
        barrier()
        check_comm()
        wall_ms = (time.perf_counter() - t0) * 1e3
        e_ms = max(ev0.elapsed_time(ev1), 0.0)
        t = torch.tensor([e_ms, wall_ms], device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e_ms = float(t[0].item())
        e2e = {"value": round(world * B * args.steps / (e_ms / 1e3), 2), "unit": "samples/s",
               "h2d_bytes_per_step": host_x[0].numel() * 4 + host_y[0].numel() * 8, "d2h_bytes_per_step": 4,
               "ms_per_step": round(e_ms / args.steps, 3), "wall_ms_per_step": round(float(t[1].item()) / args.steps, 3),
               "last_loss": round(float(loss_val), 4)}

    if rank == 0:
        value = world * B * args.steps / (ms_total / 1e3)
        rec = {
            "metric": wl["metric"],
            "value": round(value, 2), "unit": "samples/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_total / args.steps, 3), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": wl["data"],
            "config": {"model": wl["model"], "T": wl["T"], "global_batch": world * B, "per_gpu_batch": B,
                       "seq_len": wl["seq_len"], "parallelism": f"dp{world}", "optimizer": "AdamW(fused)",
                       "l2": "256 MB flush written between steps (inside the timed region)"},
            "impl": args.impl, "clocks": clocks, "last_loss": round(float(loss.item()), 4),
        }
        if e2e is not None:
            rec["e2e"] = e2e
        if n_launch is not None:
            rec["gpu_launches"] = n_launch
        rec.update(extra)
        print(json.dumps(rec))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
