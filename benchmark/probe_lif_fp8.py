#!/usr/bin/env python
"""Probe of the LIF kernel with fp8 input storage: is it available, does it agree with the fp32 kernel within the gates,
and what does it save (counterpart of the reference's ``benchmark/probe_lif_fp8_triton.py`` + ``fp8_efficiency.py``).

For each storage format (e4m3, e5m2): the input is rounded to fp8 once.  The fp8-storage kernel (bf16 spikes / states in
memory, fp32 arithmetic) is compared with the fp32 kernel on the same rounded values: spike cosine similarity >= 0.95 and
relative L2 error of the input gradient <= 0.30 are the gates (the reference's).  Also reported, without a gate: agreement
with the bf16 kernel on the widened values (storage is then the only difference) and with the fp32 kernel on the
*unrounded* input (what the rounding of the input itself costs over T steps).  Efficiency: forward + backward time of the fp8-storage kernel over the bf16 kernel (< 1 is faster).

    python benchmark/probe_lif_fp8.py [--T 64 --N 1024] [--big-N 16777216]
"""
import argparse
import json
import statistics
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent))
import _arms  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--T", type=int, default=64)
    ap.add_argument("--N", type=int, default=1024)
    ap.add_argument("--big-N", type=int, default=1 << 24, help="neurons of the timing case (T = 4)")
    ap.add_argument("--min-cosine", type=float, default=0.95)
    ap.add_argument("--max-rel-l2", type=float, default=0.30)
    a = ap.parse_args()
    _arms.load("ours")
    from spikingjelly_b200.activation_based import surrogate
    from spikingjelly_b200.activation_based.triton_kernel.neuron_kernel import multistep_lif, multistep_lif_mp
    sg = surrogate.ATan()
    torch.manual_seed(0)
    ok = True
    for name, storage in (("e4m3", torch.float8_e4m3fn), ("e5m2", torch.float8_e5m2)):
        x = (torch.randn(a.T, a.N, device="cuda") * 0.8 + 0.3)
        g = torch.randn(a.T, a.N, device="cuda")
        v0 = torch.zeros(a.N, device="cuda")
        x32 = x.clone().requires_grad_(True)
        s32, _ = multistep_lif(x32, v0, True, 2.0, 1.0, 0.0, False, sg)
        s32.backward(g)
        x8 = x.to(torch.bfloat16).requires_grad_(True)
        s8, _, _ = multistep_lif_mp(x8, v0, decay_input=True, tau=2.0, v_threshold=1.0, v_reset=0.0, storage_dtype=storage, spike_dtype=torch.bfloat16,
                                    surrogate_function=sg)
        s8.backward(g.to(torch.bfloat16))
        xw = x.to(torch.bfloat16).to(storage).to(torch.bfloat16).requires_grad_(True)
        sw, _ = multistep_lif(xw, v0.to(torch.bfloat16), True, 2.0, 1.0, 0.0, False, sg)
        sw.backward(g.to(torch.bfloat16))
        xr = x.to(torch.bfloat16).to(storage).float().requires_grad_(True)             # fp32 kernel on the rounded values
        sr, _ = multistep_lif(xr, v0, True, 2.0, 1.0, 0.0, False, sg)
        sr.backward(g)
        cosine = lambda u, v: torch.nn.functional.cosine_similarity(u.float().flatten(), v.float().flatten(), dim=0).item()
        rel_l2 = lambda u, v: ((u.float() - v.float()).norm() / v.float().norm()).item()
        cos, rel = cosine(s8, sr), rel_l2(x8.grad, xr.grad)
        passed = cos >= a.min_cosine and rel <= a.max_rel_l2
        ok &= passed
        print(json.dumps({"storage": name, "T": a.T, "N": a.N, "spike_cosine_vs_fp32_on_rounded_input": round(cos, 4),
                          "grad_rel_l2_vs_fp32_on_rounded_input": round(rel, 4), "gates": {"min_cosine": a.min_cosine, "max_rel_l2": a.max_rel_l2},
                          "passed": passed, "spike_mismatch_vs_bf16_kernel_on_widened_input": round(float((s8 != sw).float().mean()), 6),
                          "grad_rel_l2_vs_bf16_kernel_on_widened_input": round(rel_l2(x8.grad, xw.grad), 6),
                          "spike_cosine_vs_fp32_on_unrounded_input": round(cosine(s8, s32), 4), "grad_rel_l2_vs_fp32_on_unrounded_input": round(rel_l2(x8.grad, x32.grad), 4)}))
    # efficiency at a bandwidth-bound size
    T, N = 4, a.big_N
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    xb = torch.randn(T, N, device="cuda").to(torch.bfloat16).requires_grad_(True)
    gb = torch.randn(T, N, device="cuda").to(torch.bfloat16)
    v0 = torch.zeros(N, device="cuda", dtype=torch.bfloat16)
    x8 = xb.detach().to(torch.float8_e4m3fn)
    from spikingjelly_b200.ops.neuron_scan import KIND

    def bf16():
        xb.grad = None
        multistep_lif(xb, v0, True, 2.0, 1.0, 0.0, False, sg)[0].backward(gb)

    def fp8():               # the tensor already lives in fp8 (as it would after an fp8 producer): no cast in the timed region
        o = torch.ops.sjb200.scan_forward(x8, None, 0.0, None, KIND["lif_di"], 2.0, 0.0, 0.0, 0.0, 1.0, 0.0, False, False, False, True)
        torch.ops.sjb200.scan_backward(gb, None, None, x8, None, 0.0, None, o[4] if o[4].numel() else None, KIND["lif_di"], 2.0, 0.0, 0.0, 0.0, 1.0,
                                       0.0, False, 1, 2.0, 0.0, False, False)
    tb = statistics.median(_arms.time_cuda(bf16, 3, 20, flush=flush)) * 1e3
    t8 = statistics.median(_arms.time_cuda(fp8, 3, 20, flush=flush)) * 1e3
    print(json.dumps({"efficiency": {"T": T, "N": N, "bf16_us": round(tb, 1), "fp8_storage_us": round(t8, 1), "fp8_over_bf16": round(t8 / tb, 3)}, "all_gates_passed": ok}))
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
