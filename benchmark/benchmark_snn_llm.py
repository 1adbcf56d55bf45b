#!/usr/bin/env python
"""SNN-LLM (24 layers, d 2048, 16 heads, FFN 5504, vocabulary 32000, T = 4) training step: sequence length 2048,
micro-batch 4 per tensor-parallel group, random token ids, bf16 autocast, AdamW.  Tensor parallel over all ranks
(Megatron-style on NCCL); tokens/s counts the tokens of the micro-batch once (not per time step).

    python benchmark/benchmark_snn_llm.py [--layers 24 --steps 5 --warmup 2]
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 benchmark/benchmark_snn_llm.py

CUDA-event timing with a 256 MB L2 flush per step, max over ranks, one JSON line on rank 0 with the model FLOPs per
second against the measured bf16 peak.
"""
import argparse
import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
from spikingjelly_b200 import ops  # noqa: E402
from spikingjelly_b200.models import snn_llm  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--micro-batch", type=int, default=4)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--fp8", action="store_true", help="run the four linear layers of every block through the fp8 linear (TP = 1)")
    ap.add_argument("--fp8-recipe", choices=["delayed", "current"], default="delayed")
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours",
                    help="reference: the same architecture assembled from the reference package's parts (benchmark/snn_llm_reference_parts.py)")
    ap.add_argument("--path", choices=["megatron", "fused"], default="megatron",
                    help="ours, several GPUs: NCCL all-reduce tensor parallelism, or the fused token-sharded path (parallel/fused_tp_train.py)")
    ap.add_argument("--tp", type=int, default=0,
                    help="fused path: tensor-parallel group size; the remaining factor of the world is data parallel (a TP x DP mesh: "
                         "ranks [k * tp, (k + 1) * tp) form a tensor-parallel group, ranks with equal position in their group a data-parallel one)")
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    world, rank, local = (int(os.environ.get(k, d)) for k, d in (("WORLD_SIZE", "1"), ("RANK", "0"), ("LOCAL_RANK", "0")))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    torch.manual_seed(0)                                   # identical replicated parameters on every rank
    extra = {}
    sync_replicated = sync_sharded = None
    loss_scale = 1.0
    if a.impl == "reference":
        try:
            sys.path.insert(0, str(ROOT / "benchmark"))
            import snn_llm_reference_parts as ref
            backend = ref.pick_backend(device)
            model = ref.build(a.layers, a.seq, backend).to(device)
            if world > 1:
                model = ref.tensor_parallel(model, world)
            extra["reference_backend"] = backend
        except Exception as exc:
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": f"{type(exc).__name__}: {exc}"[:300]}))
            if world > 1:
                dist.destroy_process_group()
            return
    else:
        ops.require()
        model = snn_llm.snn_llm_1b(n_layers=a.layers, backend="cuda", max_seq_len=a.seq)
        if world > 1 and a.path == "megatron":
            model = snn_llm.parallelize_snn_llm(model)
        model.to(device)
        if a.path == "fused":
            from spikingjelly_b200.parallel.data_parallel import SNNDataParallel
            from spikingjelly_b200.parallel.fused_tp_train import FusedTPSNNLLM
            tp = a.tp if a.tp > 0 else world
            if world % tp:
                raise SystemExit(f"--tp {tp} does not divide the world size {world}")
            dp = world // tp
            tp_group = dp_group = None
            if dp > 1:
                # every rank creates every group (collective calls), then keeps its own two
                for k in range(dp):
                    g = dist.new_group(list(range(k * tp, (k + 1) * tp)))
                    if rank // tp == k:
                        tp_group = g
                for j in range(tp):
                    g = dist.new_group(list(range(j, world, tp)))
                    if rank % tp == j:
                        dp_group = g
            model = FusedTPSNNLLM(model, a.micro_batch, a.seq, group=tp_group)
            extra.update(tp=tp, dp=dp)
            if world > 1:
                # replicated parameters (embedding, norms, LM head) see this rank's tokens only: their gradients are summed over
                # the whole mesh; sharded parameters are summed over the data-parallel group.  The loss share is divided by dp
                # below, so both sums are the mean over data-parallel replicas of the tensor-parallel total.
                holder = torch.nn.Module()
                holder.params = torch.nn.ParameterList(model.replicated_parameters())
                sync_replicated = SNNDataParallel(holder, reduce="sum", timeout_s=120.0)
                if dp > 1:
                    replicated = {id(p) for p in holder.params}
                    sharded = torch.nn.Module()
                    sharded.params = torch.nn.ParameterList([p for p in model.parameters() if id(p) not in replicated])
                    sync_sharded = SNNDataParallel(sharded, process_group=dp_group, reduce="sum", timeout_s=120.0)
                    loss_scale = 1.0 / dp
    if a.fp8:
        # per-tensor scaled e4m3 / e5m2 operands on the tcgen05 kind::f8f6f4 GEMM in all three products (spikes are exact in
        # e4m3); the LM head stays bf16
        from spikingjelly_b200.ops import fp8
        if world > 1:
            raise SystemExit("--fp8 is wired for TP = 1 in this script")
        for blk in model.blocks:
            for lin in (blk.attn.qkv, blk.attn.proj, blk.ffn.up, blk.ffn.down):
                sc = fp8.LinearScaling() if a.fp8_recipe == "delayed" else None
                lin.forward = (lambda x, m=lin, sc=sc: fp8.linear(x, m.weight, m.bias, sc))
    # the fused AdamW kernel takes one kind of tensor per call: sharded (DTensor) and plain parameters get an optimiser each
    from torch.distributed.tensor import DTensor
    kinds = {}
    for p in model.parameters():
        kinds.setdefault(isinstance(p, DTensor) or isinstance(p.data, DTensor), []).append(p)
    opts = [torch.optim.AdamW(ps, lr=1e-4, fused=True) for ps in kinds.values()]
    replica = rank // extra["tp"] if "tp" in extra else 0           # data-parallel replicas train on different tokens
    tok = torch.randint(0, 32000, (a.micro_batch, a.seq), device=device, generator=torch.Generator(device).manual_seed(1 + replica))
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)

    def step():
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=a.path != "fused" or a.impl == "reference"):
            _, loss = model(tok, labels=tok)
        if loss_scale != 1.0:
            loss = loss * loss_scale
        for opt in opts:
            opt.zero_grad(set_to_none=True)
        loss.backward()
        for opt in opts:
            opt.step()
        flush.zero_()
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(a.warmup):
        step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        loss = step()
    e1.record()
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        ms = t.item() / a.steps
        tokens = a.micro_batch * a.seq * extra.get("dp", 1)
        fwd_flops = tokens * (model.flops_per_token(a.seq) if hasattr(model, "flops_per_token") else snn_llm.SNNLLM.flops_per_token(model, a.seq))
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
        peak = float(peaks.get("bf16_tflops_sustained", 1400.0))
        tflops = 3.0 * fwd_flops / (ms / 1e3) / 1e12 / world
        rec = {"config": f"SNN-LLM {a.layers}L d2048 ffn5504 T4 seq{a.seq} mb{a.micro_batch} {("fp8-" + a.fp8_recipe) if a.fp8 else "bf16"} tp{extra.get("tp", world)}" + (f" x dp{extra['dp']}" if extra.get("dp", 1) > 1 else ""), "n_gpus": world,
               "impl": a.impl, "path": a.path if a.impl == "ours" else "reference DTensor TP",
               "ms_per_step": round(ms, 2), "tokens_per_s": round(tokens / ms * 1e3, 1), "model_tflops_per_gpu": round(tflops, 1),
               "of_measured_sustained_bf16_peak": round(tflops / peak, 3), "peak_source": "measured" if peaks else "fallback",
               "last_loss": round(float(loss), 4), "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1),
               "parameters": sum(p.numel() for p in model.parameters())}
        rec.update(extra)
        line = json.dumps(rec)
        print(line)
        if a.out:
            with open(a.out, "a") as f:
                f.write(line + "\n")
    if sync_replicated is not None:
        sync_replicated.check_communication()
        model.check()
    if sync_sharded is not None:
        sync_sharded.check_communication()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
