#!/usr/bin/env python
"""Qwen2 ANN -> SNN conversion, correctness and time: dense logits against the converted model in ``exact_td`` and
``signed_if`` mode, cached decoding against the full pass, reset replay, the structure of the converted model, and paired
timings of the dense and the converted forward.  The role of the reference's
``benchmark/snn_llm/qwen_conversion/scaleout_smoke.py`` and ``scaleout_efficiency.py``; those load a pinned Qwen2.5 snapshot
from disk, this one builds the architecture (``--size 0.5b|1.5b|3b|tiny``, optionally fewer layers) with random weights
and random token ids, so the loss values mean nothing and the limits checked are the conversion's own: exact mode equal to
the dense model, reset replay bit-equal, cache continuation equal to the full pass.

    python benchmark/snn_llm_qwen_conversion.py [--size tiny] [--layers N] [--time-steps 16] [--device cuda] [--neuron-backend torch|cuda]
"""
import argparse
import json
import sys
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

SIZES = {      # hidden, intermediate, layers, heads, kv heads, vocabulary
    "tiny": (64, 128, 2, 4, 2, 512),
    "0.5b": (896, 4864, 24, 14, 2, 151936),
    "1.5b": (1536, 8960, 28, 12, 2, 151936),
    "3b": (2048, 11008, 36, 16, 2, 151936),
}


def relative_l2(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))


def lm_loss(logits, ids, mask):
    lp = torch.log_softmax(logits[:, :-1].float(), -1).gather(-1, ids[:, 1:, None]).squeeze(-1)
    w = mask[:, 1:].float()
    return float(-(lp * w).sum() / w.sum())


def main():
    import transformers
    from spikingjelly_b200.activation_based import functional
    from spikingjelly_b200.activation_based.ann2snn import ModuleConverter, Qwen2SNNConfig, Qwen2SNNRecipe, calibrate_qwen2_snn
    ap = argparse.ArgumentParser()
    ap.add_argument("--size", choices=sorted(SIZES), default="tiny")
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--dtype", choices=["fp32", "bf16"], default="fp32")
    ap.add_argument("--time-steps", type=int, default=16)
    ap.add_argument("--calibration-levels", type=int, default=16)
    ap.add_argument("--calibration-quantile", type=float, default=0.999)
    ap.add_argument("--neuron-backend", default=None)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq-len", type=int, default=32)
    ap.add_argument("--prefill", type=int, default=None)
    ap.add_argument("--repeats", type=int, default=3)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args()
    dev = torch.device(a.device)
    h, inter, layers, heads, kv, vocab = SIZES[a.size]
    layers = a.layers or layers
    cfg = transformers.Qwen2Config(vocab_size=vocab, hidden_size=h, intermediate_size=inter, num_hidden_layers=layers, num_attention_heads=heads,
                                   num_key_value_heads=kv, max_position_embeddings=max(2 * a.seq_len, 64), tie_word_embeddings=False)
    torch.manual_seed(a.seed)
    dense = transformers.Qwen2ForCausalLM(cfg).to(dev).eval()
    amp = torch.autocast(dev.type, dtype=torch.bfloat16, enabled=a.dtype == "bf16")
    ids = torch.randint(0, vocab, (a.batch, a.seq_len), device=dev)
    mask = torch.ones_like(ids)
    mask[0, : a.seq_len // 4] = 0                                # left padding on one row
    valid = mask.bool()
    kw = {} if a.neuron_backend is None else {"neuron_backend": a.neuron_backend}
    conf = Qwen2SNNConfig(time_steps=a.time_steps, calibration_levels=a.calibration_levels, calibration_quantile=a.calibration_quantile, **kw)
    cal_ids = torch.randint(0, vocab, (a.batch, a.seq_len), device=dev)
    with amp:
        cal = calibrate_qwen2_snn(dense, [{"input_ids": cal_ids, "attention_mask": torch.ones_like(cal_ids)}], conf)
    snn = ModuleConverter(Qwen2SNNRecipe(cal, conf)).convert(dense).eval()
    sync = (lambda: torch.cuda.synchronize(dev)) if dev.type == "cuda" else (lambda: None)

    def timed(fn):
        fn()
        sync()
        best = float("inf")
        for _ in range(a.repeats):
            t0 = time.perf_counter()
            out = fn()
            sync()
            best = min(best, time.perf_counter() - t0)
        return out, best * 1e3

    def run(mode, **extra):
        functional.reset_net(snn)
        return snn(input_ids=ids, attention_mask=mask, encoding_mode=mode, **extra).logits
    with torch.inference_mode(), amp:
        want, t_dense = timed(lambda: dense(input_ids=ids, attention_mask=mask, use_cache=False).logits)
        exact, t_exact = timed(lambda: run("exact_td"))
        signed, t_signed = timed(lambda: run("signed_if"))
        replay = run("signed_if")
        # cached decoding: prefill, then the rest token by token, against the full pass of the unpadded row
        row, pre = ids[1:], a.prefill or a.seq_len // 2
        functional.reset_net(snn)
        full = snn(input_ids=row, encoding_mode="exact_td").logits
        functional.reset_net(snn)
        out = snn(input_ids=row[:, :pre], attention_mask=torch.ones(1, pre, dtype=torch.long, device=dev), encoding_mode="exact_td", use_cache=True)
        worst_cache = relative_l2(out.logits, full[:, :pre])
        past = out.past_key_values
        for t in range(pre, a.seq_len):
            functional.reset_net(snn)
            out = snn(input_ids=row[:, t:t + 1], attention_mask=torch.ones(1, t + 1, dtype=torch.long, device=dev), encoding_mode="exact_td",
                      use_cache=True, past_key_values=past)
            past = out.past_key_values
            worst_cache = max(worst_cache, relative_l2(out.logits, full[:, t:t + 1]))
    d_loss = lm_loss(want, ids, mask)
    report = {
        "model": {"size": a.size, "hidden": h, "layers": layers, "heads": heads, "kv_heads": kv, "vocabulary": vocab,
                  "parameters": sum(p.numel() for p in dense.parameters()), "weights": "random"},
        "configuration": {"device": str(dev), "dtype": a.dtype, "time_steps": a.time_steps, "calibration_levels": a.calibration_levels,
                          "calibration_quantile": a.calibration_quantile, "neuron_backend": conf.neuron_backend, "batch": a.batch, "seq_len": a.seq_len},
        "structure": snn.structure_summary(),
        "metrics": {"dense_loss": d_loss, "exact_loss_delta": abs(lm_loss(exact, ids, mask) - d_loss),
                    "signed_loss_delta": abs(lm_loss(signed, ids, mask) - d_loss),
                    "exact_logits_relative_l2": relative_l2(exact[valid], want[valid]),
                    "signed_logits_relative_l2": relative_l2(signed[valid], want[valid]),
                    "signed_top1_agreement": float(signed.argmax(-1)[valid].eq(want.argmax(-1)[valid]).float().mean()),
                    "reset_replay_max_abs_error": float((replay.float() - signed.float()).abs().max()),
                    "exact_cached_decode_max_relative_l2": worst_cache},
        "timing_ms": {"dense_forward": round(t_dense, 3), "exact_td_forward": round(t_exact, 3), "signed_if_forward": round(t_signed, 3),
                      "signed_over_dense": round(t_signed / t_dense, 2)},
    }
    m = report["metrics"]
    tol = 1e-4 if a.dtype == "fp32" else 0.05
    report["acceptance"] = {"exact_equals_dense": m["exact_logits_relative_l2"] <= tol, "reset_replay_exact": m["reset_replay_max_abs_error"] <= 1e-6,
                            "cache_equals_full_pass": m["exact_cached_decode_max_relative_l2"] <= max(tol, 1e-4)}
    report["acceptance"]["passed"] = all(report["acceptance"].values())
    print(json.dumps(report, allow_nan=False))
    return 0 if report["acceptance"]["passed"] else 1


if __name__ == "__main__":
    sys.exit(main())
