#!/usr/bin/env python
"""Data-parallel training of a small spiking language model under each precision policy, with the invariants a distributed
mixed-precision run has to keep:

* the loss goes down over the run;
* every rank ends with bit-identical parameters (sha256 of the state dict, compared over the process group);
* after ``reset_net`` the same batch gives the same loss again (no state leaks between steps);
* a checkpoint written by rank 0 loads back into a fresh model and reproduces the evaluation loss;
* the LIF neurons run in fp32 under autocast (wrapped in ``AutocastFp32LIF`` for bf16 / fp16) and are the framework's own
  ``LIFNode`` (ownership check).

The model is a SpikeGPT-like stack (token-shift mixing, two LIF layers per block whose time axis is the token axis) built
here, because the SpikeGPT source tree the reference's ``benchmark/snn_llm/spikegpt_distributed_precision_smoke.py`` patches is
not on this machine.  The distributed side goes through ``distributed.analyze -> plan -> apply`` with ``mode="dp"``.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29571 \\
        benchmark/snn_llm_distributed_precision_smoke.py [--precisions fp32 bf16 fp16 fp8] [--device cuda|cpu]
"""
import argparse
import hashlib
import io
import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))


class AutocastFp32LIF(nn.Module):
    """Runs the wrapped neuron in fp32 with autocast off and hands the spikes back in the caller's dtype."""

    def __init__(self, lif: nn.Module):
        super().__init__()
        self.lif = lif

    @property
    def v(self):
        return self.lif.v

    def forward(self, x):
        with torch.autocast(device_type=x.device.type, enabled=False):
            y = self.lif(x.float())
        return y.to(x.dtype)


class Block(nn.Module):
    def __init__(self, dim, hidden, make_lif):
        super().__init__()
        self.ln1, self.ln2 = nn.LayerNorm(dim), nn.LayerNorm(dim)
        self.mix1, self.mix2 = nn.Parameter(torch.full((dim,), 0.5)), nn.Parameter(torch.full((dim,), 0.5))
        self.key, self.value, self.receptance, self.out = (nn.Linear(dim, dim, bias=False) for _ in range(4))
        self.up, self.down = nn.Linear(dim, hidden, bias=False), nn.Linear(hidden, dim, bias=False)
        self.lif1, self.lif2 = make_lif(), make_lif()

    @staticmethod
    def shift(x):                                   # the previous token's features (zeros for the first token)
        return F.pad(x, (0, 0, 1, -1))

    def forward(self, x):                           # [S, B, C]: the token axis is the neurons' time axis
        y = self.ln1(x)
        y = y * self.mix1 + self.shift(y.transpose(0, 1)).transpose(0, 1) * (1 - self.mix1)
        gate = torch.sigmoid(self.receptance(y))
        kv = (self.key(y).softmax(-1) * self.value(y)).cumsum(0) / torch.arange(1, x.shape[0] + 1, device=x.device, dtype=x.dtype).view(-1, 1, 1)
        x = x + self.lif1(self.out(gate * kv))
        z = self.ln2(x)
        z = z * self.mix2 + self.shift(z.transpose(0, 1)).transpose(0, 1) * (1 - self.mix2)
        return x + self.lif2(self.down(F.relu(self.up(z)) ** 2))


class SpikingLM(nn.Module):
    def __init__(self, vocab, dim, hidden, layers, make_lif):
        super().__init__()
        self.emb = nn.Embedding(vocab, dim)
        self.blocks = nn.ModuleList(Block(dim, hidden, make_lif) for _ in range(layers))
        self.ln_out, self.head = nn.LayerNorm(dim), nn.Linear(dim, vocab, bias=False)

    def forward(self, ids):                         # [B, S] -> [B, S, V]
        x = self.emb(ids).transpose(0, 1)
        for b in self.blocks:
            x = b(x)
        return self.head(self.ln_out(x)).transpose(0, 1)


def state_digest(model: nn.Module) -> str:
    h = hashlib.sha256()
    for k, v in sorted(model.state_dict().items()):
        h.update(k.encode())
        h.update(v.detach().cpu().contiguous().view(torch.uint8).numpy().tobytes())
    return h.hexdigest()


def unwrap(m):
    while hasattr(m, "module"):
        m = m.module
    return m


def main():
    from spikingjelly_b200.activation_based import distributed as sjd, functional, neuron, precision, surrogate
    ap = argparse.ArgumentParser()
    ap.add_argument("--precisions", nargs="+", default=["fp32", "bf16", "fp16", "fp8"])
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--batch", type=int, default=8, help="per rank")
    ap.add_argument("--seq-len", type=int, default=32)
    ap.add_argument("--vocab", type=int, default=256)
    ap.add_argument("--dim", type=int, default=128)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--lr", type=float, default=3e-3)
    ap.add_argument("--clip", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=1234)
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    cuda = a.device == "cuda"
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(dev)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl" if cuda else "gloo")
    backend = "cuda" if cuda else "torch"
    sg = surrogate.ATan()
    make_lif = lambda: neuron.LIFNode(tau=2.0, surrogate_function=sg, step_mode="m", backend=backend)    # noqa: E731
    # a byte-level corpus with structure: every row repeats a short random motif, so a few steps already lower the loss
    g = torch.Generator().manual_seed(a.seed)
    motifs = torch.randint(0, a.vocab, (64, 8), generator=g)

    def batch(step, r):
        gi = torch.Generator().manual_seed(a.seed * 1000 + step * 97 + r)
        rows = motifs[torch.randint(0, 64, (a.batch,), generator=gi)]
        return rows.repeat(1, a.seq_len // 8 + 1)[:, : a.seq_len + 1].to(dev)
    reports = []
    for mode in a.precisions:
        row = {"precision": mode, "world_size": world}
        try:
            torch.manual_seed(a.seed)
            net = SpikingLM(a.vocab, a.dim, 4 * a.dim, a.layers, make_lif).to(dev)
            if mode in ("bf16", "fp16"):
                for b in net.blocks:
                    b.lif1, b.lif2 = AutocastFp32LIF(b.lif1), AutocastFp32LIF(b.lif2)
            lifs = [m for m in net.modules() if isinstance(m, neuron.LIFNode)]
            row["lif_nodes"] = len(lifs)
            row["lif_ownership_ok"] = len(lifs) == 2 * a.layers and all(type(m).__module__.startswith("spikingjelly_b200.") for m in lifs)
            art = precision.prepare_model_for_precision(net, dev, precision.PrecisionConfig(mode=mode, strictness="warn" if mode == "fp8" else "strict",
                                                                                           device=str(dev)))
            net = art.model
            row["effective_mode"] = art.effective_config.mode
            if world > 1:
                plan = sjd.plan(analysis=sjd.analyze(net), objective="speed", topology={"dp": world}, backend=backend, batch_size=a.batch,
                                model_family=None, mode="dp")
                runtime = sjd.apply(model=net, plan=plan, device_type=dev.type)
                net = runtime.model
            opt = torch.optim.AdamW(unwrap(net).parameters(), lr=a.lr)

            def loss_of(tokens):
                with art.autocast_context():
                    logits = net(tokens[:, :-1])
                return F.cross_entropy(logits.float().flatten(0, 1), tokens[:, 1:].flatten())
            losses = []
            for step in range(a.steps):
                opt.zero_grad(set_to_none=True)
                loss = loss_of(batch(step, rank))
                art.backward(loss, opt, clip_grad_norm=a.clip, parameters=unwrap(net).parameters())
                functional.reset_net(net)
                losses.append(float(loss.detach()))
            k = max(1, a.steps // 5)
            row["first_losses"], row["last_losses"] = round(sum(losses[:k]) / k, 4), round(sum(losses[-k:]) / k, 4)
            row["loss_decreased"] = row["last_losses"] < row["first_losses"]
            net.eval()
            with torch.no_grad():
                probe = batch(10_000, 0)
                e1 = float(loss_of(probe))
                functional.reset_net(net)
                e2 = float(loss_of(probe))
                functional.reset_net(net)
            row["reset_replay_equal"] = e1 == e2
            digest = state_digest(unwrap(net))
            if world > 1:
                all_d = [None] * world
                dist.all_gather_object(all_d, digest)
                row["ranks_identical"] = len(set(all_d)) == 1
            row["state_sha256"] = digest[:16]
            # checkpoint round trip (rank 0 writes to memory, every rank loads the broadcast bytes)
            buf = io.BytesIO()
            if rank == 0:
                torch.save(unwrap(net).state_dict(), buf)
            blob = [buf.getvalue()]
            if world > 1:
                dist.broadcast_object_list(blob, src=0)
            torch.manual_seed(a.seed + 1)
            fresh = SpikingLM(a.vocab, a.dim, 4 * a.dim, a.layers, make_lif).to(dev)
            if mode in ("bf16", "fp16"):
                for b in fresh.blocks:
                    b.lif1, b.lif2 = AutocastFp32LIF(b.lif1), AutocastFp32LIF(b.lif2)
            fresh_art = precision.prepare_model_for_precision(fresh, dev, precision.PrecisionConfig(
                mode=mode, strictness="warn" if mode == "fp8" else "strict", device=str(dev)))
            fresh_art.model.load_state_dict(torch.load(io.BytesIO(blob[0]), map_location=dev, weights_only=True))
            fresh_art.model.eval()
            with torch.no_grad(), fresh_art.autocast_context():
                e3 = float(F.cross_entropy(fresh_art.model(probe[:, :-1]).float().flatten(0, 1), probe[:, 1:].flatten()))
            row["checkpoint_eval_loss_delta"] = abs(e3 - e1)
            row["checkpoint_reproduces"] = row["checkpoint_eval_loss_delta"] <= (1e-6 if mode == "fp32" else 5e-3)
            row["passed"] = all(row.get(k, True) for k in ("lif_ownership_ok", "loss_decreased", "reset_replay_equal", "ranks_identical", "checkpoint_reproduces"))
        except Exception as exc:
            row["unavailable"] = f"{type(exc).__name__}: {exc}"[:240]
        reports.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    bad = [r["precision"] for r in reports if r.get("passed") is False]
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
