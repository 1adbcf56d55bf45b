#!/usr/bin/env python
"""Neuron-kernel sweep: multi-step IF / LIF / PLIF forward+backward on one GPU.

For every (neuron, reset, dtype, T, N) it times forward+backward of
  * ours:      spikingjelly_b200 native kernels (backend="cuda")
  * reference: the unmodified reference's torch and triton backends (from baseline/_ref),
and reports microseconds, achieved GB/s against the algorithmic traffic of OUR kernels
(read x, write spikes; read x, read grad, write grad_x) and the speed-up over the
reference's fastest backend.  Inputs x ~ N(0.5, 1), upstream gradients ~ N(0, 1); each
timed iteration follows an L2 flush; CUDA-event timing after warm-up.

    python benchmark/benchmark_neuron_kernels.py --out out/neuron_sweep.json
"""
import argparse
import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))


def time_fn(fn, flush, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2] * 1e3  # us


def make(ns, kind, soft, backend):
    kw = dict(v_reset=None if soft else 0.0, surrogate_function=ns.surrogate.ATan(), step_mode="m", backend=backend)
    if kind == "if":
        return ns.neuron.IFNode(**kw)
    if kind == "lif":
        return ns.neuron.LIFNode(tau=2.0, decay_input=True, **kw)
    if kind == "lif_ndi":
        return ns.neuron.LIFNode(tau=2.0, decay_input=False, **kw)
    return ns.neuron.ParametricLIFNode(init_tau=2.0, **kw)


def headline(args, dev):
    T, N = 4, 1 << 24
    x = (torch.randn(T, N, device=dev) + 0.5).to(torch.bfloat16).requires_grad_(True)
    g = torch.randn(T, N, device=dev).to(torch.bfloat16)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    class NS:
        pass
    rec = {"neuron": "lif", "soft_reset": False, "dtype": "bf16", "T": T, "N": N, "impl": args.impl}
    if args.impl == "ours":
        from spikingjelly_b200 import ops
        from spikingjelly_b200.activation_based import functional, neuron, surrogate
        ops.require()
        NS.neuron, NS.surrogate, NS.functional = neuron, surrogate, functional
        backends = ["cuda"]
    else:
        try:
            sys.path.insert(0, str(ROOT / "baseline" / "_ref"))
            from spikingjelly.activation_based import functional as rf, neuron as rn, surrogate as rs
        except Exception as exc:
            print(json.dumps({"impl": "reference", "unavailable": f"{type(exc).__name__}: {exc}"[:300]}))
            return
        NS.neuron, NS.surrogate, NS.functional = rn, rs, rf
        backends = args.ref_backends.split(",")
    times = {}
    for be in backends:
        try:
            net = make(NS, "lif", False, be).to(dev)

            def f():
                x.grad = None
                net(x).backward(g)
                NS.functional.reset_net(net)
            times[be] = round(time_fn(f, flush, iters=args.iters), 2)
        except Exception as exc:
            rec[f"{be}_err"] = f"{type(exc).__name__}: {exc}"[:120]
    if not times:
        print(json.dumps({"impl": args.impl, "unavailable": "no neuron backend ran: " + "; ".join(str(v) for k, v in rec.items() if k.endswith("_err"))}))
        return
    best = min(times, key=times.get)
    rec.update(fwd_bwd_us=times[best], backend=best, all_backends_us=times,
               GBps=round(5 * T * N * 2 / times[best] / 1e3, 1))
    print(json.dumps(rec))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="")
    ap.add_argument("--T", default="4,8,16,32")
    ap.add_argument("--logN", default="16,20,24")
    ap.add_argument("--dtypes", default="fp32,bf16")
    ap.add_argument("--neurons", default="if,lif,lif_ndi,plif")
    ap.add_argument("--no-reference", action="store_true")
    ap.add_argument("--ref-backends", default="torch,triton")
    ap.add_argument("--headline", action="store_true",
                    help="one record only: LIF (tau 2, hard reset, ATan) forward + backward, bf16, T = 4, N = 2^24, for --impl")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--bits", action="store_true", help="also time the bit-only spike output (ours) and the reference's dense kernel + "
                    "BitSpikeCompressor")
    args = ap.parse_args()
    dev = torch.device("cuda")
    if args.headline:
        return headline(args, dev)
    from spikingjelly_b200.activation_based import functional, neuron, surrogate

    class Ours:
        pass
    Ours.neuron, Ours.surrogate, Ours.functional = neuron, surrogate, functional
    Ref = None
    if not args.no_reference:
        try:
            sys.path.insert(0, str(ROOT / "baseline" / "_ref"))
            from spikingjelly.activation_based import functional as rf, neuron as rn, surrogate as rs

            class Ref:
                pass
            Ref.neuron, Ref.surrogate, Ref.functional = rn, rs, rf
        except Exception as exc:
            print("reference unavailable:", exc, file=sys.stderr)
    dts = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16, "fp8": torch.bfloat16}
    from spikingjelly_b200 import ops
    from spikingjelly_b200.ops.neuron_scan import KIND
    ops.require()
    kind_id = {"if": KIND["if"], "lif": KIND["lif_di"], "lif_ndi": KIND["lif_ndi"]}
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows = []
    for kind in args.neurons.split(","):
        for soft in (False, True):
            for dname in args.dtypes.split(","):
                dt = dts[dname]
                for T in map(int, args.T.split(",")):
                    for logn in map(int, args.logN.split(",")):
                        N = 1 << logn
                        x = (torch.randn(T, N, device=dev) + 0.5).to(dt).requires_grad_(True)
                        g = torch.randn(T, N, device=dev).to(dt)

                        def run(net, ns):
                            def f():
                                x.grad = None
                                net(x).backward(g)
                                ns.functional.reset_net(net)
                            return f
                        row = {"neuron": kind, "soft_reset": soft, "dtype": dname, "T": T, "N": N}
                        if dname == "fp8":
                            # x is stored as e4m3 (1 byte); spikes and gradients are bf16.  The reference column is its
                            # mixed-precision LIF (`multistep_lif_mp`: fp8 storage, fp32 compute, bf16 spikes), which exists for
                            # LIF only; IF rows keep the reference's bf16 kernels on the widened values.
                            if kind not in kind_id:
                                continue
                            x8 = x.detach().to(torch.float8_e4m3fn)
                            k, vr = kind_id[kind], 0.0

                            def ours_fp8():
                                o = torch.ops.sjb200.scan_forward(x8, None, 0.0, None, k, 2.0, 0.0, 0.0, 0.0, 1.0, vr, soft, False, False, True)
                                torch.ops.sjb200.scan_backward(g, None, None, x8, None, 0.0, None, o[4] if o[4].numel() else None, k, 2.0,
                                                               0.0, 0.0, 0.0, 1.0, vr, soft, 1, 2.0, 0.0, False, False)
                            row["ours_us"] = round(time_fn(ours_fp8, flush), 2)
                            bytes_moved = T * N * (1 + 2 + 1 + 2 + 2)
                        else:
                            net = make(Ours, kind, soft, "cuda").to(dev)
                            row["ours_us"] = round(time_fn(run(net, Ours), flush), 2)
                            bytes_moved = 5 * T * N * x.element_size()
                            if args.bits and kind in kind_id:
                                # forward emits only bit-packed spikes (1/8 byte per element); backward is unchanged
                                from spikingjelly_b200.ops import bitspike
                                from spikingjelly_b200.ops.neuron_scan import NeuronSpec
                                spec = NeuronSpec(kind=kind_id[kind], v_threshold=1.0, v_reset=None if soft else 0.0, tau=2.0, sg=(1, 2.0, 0.0))

                                def ours_bits():
                                    x.grad = None
                                    bits, _ = bitspike.multistep_neuron_bits(x, 0.0, spec)
                                    bits.handle.backward(g)
                                row["ours_bits_us"] = round(time_fn(ours_bits, flush), 2)
                                if Ref is not None:
                                    try:
                                        # the reference's way to keep spikes as bits: its memopt compressor after the dense kernel
                                        from spikingjelly.activation_based.memopt.compress import BitSpikeCompressor
                                        rnet = make(Ref, kind, soft, "triton").to(dev)
                                        comp = BitSpikeCompressor()

                                        def ref_bits():
                                            x.grad = None
                                            s = rnet(x)
                                            comp.compress(s.detach())
                                            s.backward(g)
                                            Ref.functional.reset_net(rnet)
                                        row["ref_triton_bitcompress_us"] = round(time_fn(ref_bits, flush, iters=5, warmup=2), 2)
                                    except Exception as exc:
                                        row["ref_triton_bitcompress_err"] = f"{type(exc).__name__}: {exc}"[:160]
                        row["ours_GBps"] = round(bytes_moved / row["ours_us"] / 1e3, 1)
                        if Ref is not None and dname == "fp8" and kind in ("lif", "lif_ndi"):
                            try:
                                from spikingjelly.activation_based.triton_kernel.neuron_kernel.lif import multistep_lif_mp
                                sgf = Ref.surrogate.ATan()
                                v0 = torch.zeros(N, device=dev, dtype=torch.bfloat16)

                                def ref_mp():
                                    x.grad = None
                                    out = multistep_lif_mp(x, v0, decay_input=(kind == "lif"), tau=2.0, v_threshold=1.0, v_reset=None if soft else 0.0,
                                                           storage_dtype=torch.float8_e4m3fn, compute_dtype="fp32", backward_compute_dtype="fp32",
                                                           spike_dtype=torch.bfloat16, surrogate_function=sgf)
                                    out[0].backward(g)
                                row["ref_triton_mp_fp8_us"] = round(time_fn(ref_mp, flush, iters=5, warmup=2), 2)
                            except Exception as exc:
                                row["ref_triton_mp_fp8_err"] = f"{type(exc).__name__}: {exc}"[:160]
                        if Ref is not None:
                            for be in args.ref_backends.split(","):
                                if be == "torch" and T * N > (1 << 27):
                                    continue
                                try:
                                    rnet = make(Ref, kind, soft, be).to(dev)
                                    row[f"ref_{be}_us"] = round(time_fn(run(rnet, Ref), flush, iters=5, warmup=2), 2)
                                except Exception as exc:
                                    row[f"ref_{be}_err"] = f"{type(exc).__name__}: {exc}"[:120]
                            best = min([row[k] for k in row if k.startswith("ref_") and k.endswith("_us")], default=None)
                            if best:
                                row["speedup_vs_best_ref"] = round(best / row["ours_us"], 2)
                        print(json.dumps(row), flush=True)
                        rows.append(row)
                        del x, g
    if args.out:
        Path(args.out).parent.mkdir(parents=True, exist_ok=True)
        Path(args.out).write_text(json.dumps(rows, indent=1))


if __name__ == "__main__":
    main()
