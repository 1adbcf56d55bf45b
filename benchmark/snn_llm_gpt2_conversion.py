#!/usr/bin/env python
"""Three small causal-LM checks on a GPT-2 architecture with random weights (no snapshot is loaded):

``dense``   loss and perplexity of the dense model on the fixed synthetic batch: the number the other two compare with
``mlp``     the activation behind the GELU of one block is sent through a signed dual-channel IF encoder
            (``SignedQCFSSequenceEncoder``, T steps, per-channel symmetric scale = absmax / T) by a ``ModuleConverter`` recipe
            that swaps that block's MLP; reported: IF counts equal to the QCFS quantiser, relative L2 of the hidden
            activation and of the logits, loss change, spike rates
``cache``   prefill + token-by-token decoding with the key/value cache against one full pass (logits relative L2)

The role of the reference's ``benchmark/snn_llm/gpt2_conversion/{dense_baseline,mlp_ann2snn_slice,cache_equivalence}.py``.

    python benchmark/snn_llm_gpt2_conversion.py [--check dense mlp cache] [--layers 2] [--device cuda]
"""
import argparse
import json
import math
import sys
from pathlib import Path

import torch
import torch.nn as nn

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))


def relative_l2(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))


def lm_loss(logits, ids):
    return float(nn.functional.cross_entropy(logits[:, :-1].float().flatten(0, 1), ids[:, 1:].flatten()))


class SignedIFMLP(nn.Module):
    """GPT-2 MLP whose hidden activation (behind the GELU) passes through the signed IF encoder before ``c_proj``."""

    def __init__(self, mlp: nn.Module, encoder: nn.Module):
        super().__init__()
        self.c_fc, self.act, self.c_proj, self.encoder = mlp.c_fc, mlp.act, mlp.c_proj, encoder
        self.last_dense = self.last_if = None

    def forward(self, x):
        self.last_dense = self.act(self.c_fc(x))
        self.last_if = self.encoder.encode(self.last_dense).sum(0)
        return self.c_proj(self.last_if)


def main():
    import transformers
    from spikingjelly_b200.activation_based.ann2snn import ModuleConverter, ModuleConversionRecipe, SignedQCFSSequenceEncoder

    class GPT2MLPSignedIFRecipe(ModuleConversionRecipe):
        def __init__(self, scale: torch.Tensor, time_steps: int):
            self.scale, self.time_steps = scale.detach(), time_steps

        def validate(self, converter) -> None:
            if self.time_steps <= 0:
                raise ValueError("time_steps must be positive.")

        def convert_module(self, converter, ann: nn.Module) -> nn.Module:
            if not isinstance(getattr(ann, "c_proj", None), nn.Module):
                raise TypeError("GPT-2 MLP must expose a c_proj module.")
            return SignedIFMLP(ann, SignedQCFSSequenceEncoder(self.scale, self.time_steps, name="gpt2_mlp"))
    ap = argparse.ArgumentParser()
    ap.add_argument("--check", nargs="+", choices=["dense", "mlp", "cache"], default=["dense", "mlp", "cache"])
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--layers", type=int, default=2, help="GPT-2 small has 12")
    ap.add_argument("--hidden", type=int, default=768)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--vocab", type=int, default=50257)
    ap.add_argument("--max-samples", type=int, default=4)
    ap.add_argument("--max-length", type=int, default=64)
    ap.add_argument("--block-index", type=int, default=0)
    ap.add_argument("--time-steps", type=int, default=16)
    ap.add_argument("--prefill-length", type=int, default=16)
    ap.add_argument("--decode-steps", type=int, default=8)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args()
    dev = torch.device(a.device)
    torch.manual_seed(a.seed)
    cfg = transformers.GPT2Config(vocab_size=a.vocab, n_positions=max(a.max_length, 64), n_embd=a.hidden, n_layer=a.layers, n_head=a.heads,
                                  resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    model = transformers.GPT2LMHeadModel(cfg).to(dev).eval()
    ids = torch.randint(0, a.vocab, (a.max_samples, a.max_length), device=dev)
    report = {"model": {"architecture": "gpt2", "layers": a.layers, "hidden": a.hidden, "heads": a.heads, "vocabulary": a.vocab,
                        "parameters": sum(p.numel() for p in model.parameters()), "weights": "random"},
              "device": str(dev), "samples": a.max_samples, "length": a.max_length}
    with torch.inference_mode():
        dense_logits = model(input_ids=ids, use_cache=False).logits
        dense_loss = lm_loss(dense_logits, ids)
        if "dense" in a.check:
            report["dense"] = {"loss": dense_loss, "perplexity": math.exp(min(dense_loss, 50.0)), "tokens": int(ids[:, 1:].numel())}
        if "mlp" in a.check:
            block = model.transformer.h[a.block_index]
            grabbed = {}
            hook = block.mlp.act.register_forward_hook(lambda m, i, o: grabbed.__setitem__("h", o.detach()))
            model(input_ids=ids, use_cache=False)
            hook.remove()
            hidden = grabbed["h"]
            scale = hidden.abs().amax(dim=(0, 1)).clamp_min(1e-6) / a.time_steps
            qcfs = torch.round(hidden / scale).clamp(-a.time_steps, a.time_steps) * scale
            dense_mlp = block.mlp
            block.mlp = ModuleConverter(recipe=GPT2MLPSignedIFRecipe(scale, a.time_steps), device=dev).convert(dense_mlp)
            try:
                snn_logits = model(input_ids=ids, use_cache=False).logits
                enc = block.mlp.encoder
                report["mlp"] = {"block_index": a.block_index, "time_steps": a.time_steps, "calibration": "per_channel_symmetric_absmax",
                                 "if_vs_qcfs_max_abs_error": float((block.mlp.last_if - qcfs).abs().max()),
                                 "hidden_relative_l2": relative_l2(block.mlp.last_if, hidden),
                                 "logits_relative_l2": relative_l2(snn_logits, dense_logits),
                                 "loss_delta": abs(lm_loss(snn_logits, ids) - dense_loss),
                                 "top1_agreement": float(snn_logits.argmax(-1).eq(dense_logits.argmax(-1)).float().mean()),
                                 "positive_spike_rate": enc.positive_spike_rate, "negative_spike_rate": enc.negative_spike_rate,
                                 "boundary_correction_fraction": enc.boundary_correction_fraction}
            finally:
                block.mlp = dense_mlp
        if "cache" in a.check:
            pre, steps = a.prefill_length, min(a.decode_steps, a.max_length - a.prefill_length)
            out = model(input_ids=ids[:, :pre], use_cache=True)
            worst, past = relative_l2(out.logits, dense_logits[:, :pre]), out.past_key_values
            for t in range(pre, pre + steps):
                out = model(input_ids=ids[:, t:t + 1], past_key_values=past, use_cache=True)
                past = out.past_key_values
                worst = max(worst, relative_l2(out.logits, dense_logits[:, t:t + 1]))
            report["cache"] = {"prefill_length": pre, "decode_steps": steps, "max_logits_relative_l2": worst, "equivalent": worst <= 1e-3}
    ok = report.get("cache", {}).get("equivalent", True) and report.get("mlp", {}).get("if_vs_qcfs_max_abs_error", 0.0) <= 1e-5
    report["acceptance"] = {"passed": bool(ok)}
    print(json.dumps(report, allow_nan=False))
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
