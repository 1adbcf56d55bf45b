#!/usr/bin/env python
"""Deterministic smoke workload for the SNN-LLM family: a tiny model (``models.snn_llm.snn_llm_tiny``), fixed seed, a few
AdamW steps on a fixed synthetic token stream, and a JSON record of what ran: environment, settings, loss trajectory and
a checksum of the final parameters.  Two runs on the same machine and device must write the same ``result`` block; the
script verifies that itself with ``--repeat 2``.  Counterpart of the reference's ``benchmark/snn_llm/smoke.py`` (a
provenance-recording smoke run), on this framework's own model.

    python benchmark/snn_llm_smoke.py --device cpu --output-dir gpurun_out/snn_llm_smoke [--repeat 2]
"""
import argparse
import datetime as dt
import hashlib
import json
import platform
import sys
import uuid
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
from spikingjelly_b200.activation_based import functional  # noqa: E402
from spikingjelly_b200.models import snn_llm  # noqa: E402

SCHEMA_VERSION = 1
SEED, BATCH, SEQ, STEPS, LR = 20260713, 2, 16, 8, 1e-2


def run_once(device: torch.device) -> dict:
    torch.manual_seed(SEED)
    model = snn_llm.snn_llm_tiny(backend="cuda" if device.type == "cuda" else "torch", max_seq_len=SEQ).to(device)
    vocab = model.cfg.vocab_size
    tokens = torch.randint(0, vocab, (BATCH, SEQ), generator=torch.Generator().manual_seed(SEED + 1)).to(device)
    opt = torch.optim.AdamW(model.parameters(), lr=LR)
    losses = []
    for _ in range(STEPS):
        functional.reset_net(model)
        _, loss = model(tokens, labels=tokens)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    digest = hashlib.sha256()
    for name, p in sorted(model.state_dict().items()):
        digest.update(name.encode())
        digest.update(p.detach().float().cpu().numpy().tobytes())
    return {"losses": [round(v, 6) for v in losses], "loss_decreased": losses[-1] < losses[0], "parameter_sha256": digest.hexdigest(),
            "parameters": sum(p.numel() for p in model.parameters())}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", choices=("cpu", "cuda"), required=True)
    ap.add_argument("--output-dir", type=Path, required=True)
    ap.add_argument("--repeat", type=int, default=1)
    a = ap.parse_args()
    device = torch.device(a.device)
    if device.type == "cuda":
        from spikingjelly_b200 import ops
        ops.require()
    runs = [run_once(device) for _ in range(max(1, a.repeat))]
    record = {"schema_version": SCHEMA_VERSION, "run_id": uuid.uuid4().hex, "utc": dt.datetime.now(dt.timezone.utc).isoformat(timespec="seconds"),
              "settings": {"seed": SEED, "batch": BATCH, "sequence_length": SEQ, "steps": STEPS, "lr": LR, "device": a.device},
              "environment": {"python": platform.python_version(), "torch": torch.__version__, "platform": platform.platform(),
                              "gpu": torch.cuda.get_device_name(0) if device.type == "cuda" else None},
              "result": runs[0], "reproducible": all(r == runs[0] for r in runs), "repeats": len(runs)}
    a.output_dir.mkdir(parents=True, exist_ok=True)
    path = a.output_dir / "snn_llm_smoke.json"
    path.write_text(json.dumps(record, indent=2))
    print(json.dumps({"written": str(path), "reproducible": record["reproducible"], "loss_first": runs[0]["losses"][0],
                      "loss_last": runs[0]["losses"][-1]}))
    return 0 if record["reproducible"] and runs[0]["loss_decreased"] else 1


if __name__ == "__main__":
    sys.exit(main())
