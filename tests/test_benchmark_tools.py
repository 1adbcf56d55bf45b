"""The benchmark folder's host-side tools: the record analyser and the deterministic SNN-LLM smoke run."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT / "benchmark"))


def _records(tmp_path):
    rows = []
    for impl, base in (("ours", 1000.0), ("reference", 250.0)):
        for n in (1, 2, 8):
            for trial in range(3):
                rows.append({"impl": impl, "model": "m", "n_gpus": n, "samples_per_s": base * n * (0.95 if n > 1 else 1.0) + trial, "step_ms": 1.0})
    path = tmp_path / "r.jsonl"
    path.write_text("header line that is not json\n" + "\n".join(json.dumps(r) for r in rows))
    return path


def test_group_compare_and_scaling(tmp_path, capsys):
    import analyze_distributed_benchmark as A
    path = _records(tmp_path)
    rows = A.load_records(str(path))
    assert len(rows) == 18
    table = A.group_and_aggregate(rows, ["impl", "n_gpus"], ["samples_per_s"])
    assert len(table) == 6 and table[0]["count"] == 3 and table[0]["samples_per_s.median"] == 1001.0
    cmp_rows = A.compare(rows, ["model", "n_gpus"], "impl", "ours", "reference", "samples_per_s")
    assert len(cmp_rows) == 3 and all(3.9 < r["ratio"] < 4.1 for r in cmp_rows)
    sc = A.scaling(A.filter_records(rows, {"impl": "ours"}), ["model"], "n_gpus", "samples_per_s")
    assert [r["n_gpus"] for r in sc] == [1, 2, 8] and sc[0]["efficiency"] == 1.0 and 0.94 < sc[2]["efficiency"] < 0.96
    assert A.main([str(path), "--group-by", "impl,n_gpus", "--metric", "samples_per_s", "--format", "csv"]) == 0
    out = capsys.readouterr().out
    assert out.splitlines()[0].startswith("impl,n_gpus,count") and len(out.strip().splitlines()) == 7
    assert A.main([str(path), "--group-by", "model,n_gpus", "--compare", "impl=ours:reference", "--metric", "samples_per_s"]) == 0
    assert "ratio" in capsys.readouterr().out


def test_snn_llm_smoke_is_reproducible(tmp_path):
    r = subprocess.run([sys.executable, str(ROOT / "benchmark" / "snn_llm_smoke.py"), "--device", "cpu", "--output-dir", str(tmp_path), "--repeat", "2"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    rec = json.loads((tmp_path / "snn_llm_smoke.json").read_text())
    assert rec["reproducible"] and rec["result"]["loss_decreased"] and len(rec["result"]["parameter_sha256"]) == 64


def _json_line(args):
    r = subprocess.run([sys.executable, *args], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    return json.loads(r.stdout.strip().splitlines()[-1])


def test_ann2snn_benchmarks_run_on_cpu():
    small = ["--device", "cpu", "--time-steps", "4", "--batch-size", "2", "--batches-per-epoch", "1", "--epochs", "1", "--warmup-epochs", "0",
             "--num-classes", "10"]
    d = _json_line([str(ROOT / "benchmark" / "benchmark_ann2snn_step_mode.py"), "--recipe", "rate", "--channels", "8", "--conv-depth", "2", "--hidden-dim", "16",
                    "--image-size", "16", *small])
    assert d["parity_max_abs_diff"] <= 1e-5 and d["multi_step_speedup"] > 0
    d = _json_line([str(ROOT / "benchmark" / "benchmark_ann2snn_step_mode.py"), "--recipe", "sta", "--embed-dim", "16", "--mlp-dim", "32", "--depth", "1",
                    "--num-heads", "2", "--seq-len", "4", "--input-dim", "8", *small])
    assert d["parity_max_abs_diff"] <= 1e-4
    d = _json_line([str(ROOT / "benchmark" / "benchmark_ann2snn_spikezip_stbif.py"), "--device", "cpu", "--numel", "512", "--repeat", "1", "--sym"])
    assert d["torch_max_abs_diff"] == 0 and d["torch_state_max_abs_diff"] == 0 and d["sum_equals_quantiser"]
    d = _json_line([str(ROOT / "benchmark" / "benchmark_ann2snn_spikezip_vit_qann.py"), "--device", "cpu", "--dim", "16", "--depth", "1", "--heads", "2",
                    "--image-size", "32", "--time-steps", "48", "--batches", "1"])
    assert d["top1_agreement"] >= 0.5 and d["logit_max_abs_diff"] < 1.0


def test_fp8_efficiency_gates():
    import pytest
    import fp8_efficiency as E
    base = {"precision": "bf16", "training_samples_per_sec": 100.0, "inference_samples_per_sec": 200.0, "training_peak_allocated_mb": 10.0,
            "inference_peak_allocated_mb": 4.0}
    fast = {**base, "precision": "fp8", "training_samples_per_sec": 120.0, "inference_samples_per_sec": 260.0, "training_peak_allocated_mb": 9.0}
    slow = {**base, "precision": "fp8-b", "training_samples_per_sec": 101.0}
    rep = E.assess_model_efficiency([base, fast, slow], baseline_precision="bf16", min_training_speedup=1.05, min_inference_speedup=1.05)
    assert not rep["passed"] and rep["comparisons"][0]["passed"] and rep["comparisons"][0]["training_memory_ratio"] == 0.9
    assert len(rep["failures"]) == 2 and "fp8-b training speedup 1.0100x" in rep["failures"][0]
    with pytest.raises(RuntimeError, match="fp8-b"):
        E.require_efficiency(rep)
    E.require_efficiency(E.assess_model_efficiency([base, fast], baseline_precision="bf16", min_training_speedup=1.05, min_inference_speedup=1.05))
    for bad in ([fast], [base], [base, base, fast], [base, {**fast, "training_samples_per_sec": float("nan")}]):
        with pytest.raises(ValueError):
            E.assess_model_efficiency(bad, baseline_precision="bf16", min_training_speedup=1.05, min_inference_speedup=1.05)
    with pytest.raises(ValueError):
        E.assess_model_efficiency([base, fast], baseline_precision="fp8", min_training_speedup=1.0, min_inference_speedup=1.0)
    g = {"T": 4, "N": 1024, "neuron_type": "lif", "process": "training"}
    rows = [{**g, "variant": "stable_fp32", "success": True, "median_ms": 2.0, "peak_allocated_mb": 8.0},
            {**g, "variant": "mp_plan_float8_e4m3fn", "success": True, "median_ms": 1.0, "peak_allocated_mb": 2.0, "compute_dtype": "fp32"},
            {**g, "variant": "mp_plan_float8_e5m2", "success": True, "median_ms": 1.6, "peak_allocated_mb": 2.0},
            {**g, "T": 8, "variant": "mp_plan_float8_e5m2", "success": True, "median_ms": 1.6, "peak_allocated_mb": 2.0},
            {**g, "N": 64, "variant": "stable_fp32", "success": False, "failure_reason": "boom"}]
    rep = E.assess_triton_efficiency(rows, min_speedup=1.05)
    assert rep["comparisons"] == [{**g, "baseline_variant": "stable_fp32", "best_fp8_variant": "mp_plan_float8_e4m3fn", "best_compute_dtype": "fp32",
                                   "speedup": 2.0, "memory_ratio": 0.25, "passed": True}]
    assert len(rep["failures"]) == 2 and "boom" in rep["failures"][0] and "T=8" in rep["failures"][1]
    assert E.percentile([1.0, 3.0], 0.5) == 2.0


def test_precision_sweep_collects_rows_and_ratios():
    import benchmark_train_precision_snn_fc_sweep as S
    rows = S.collect(["noise", json.dumps({"precision": "fp32", "train_ms": 4.0}), json.dumps({"precision": "bf16", "train_ms": 2.0}),
                      json.dumps({"precision": "fp8", "train_ms": 1.6}), "{broken", json.dumps({"other": 1})])
    assert set(rows) == {"fp32", "bf16", "fp8"}
    assert S.ratios(rows) == {"bf16_over_fp32_speedup": 2.0, "fp8_over_bf16_speedup": 1.25}
    import pytest
    with pytest.raises(ValueError):
        S.main(["--hidden-dims", "100"])


def test_snn_llm_conversion_runners_on_cpu():
    import pytest
    pytest.importorskip("transformers")
    d = _json_line([str(ROOT / "benchmark" / "snn_llm_qwen_conversion.py"), "--device", "cpu", "--time-steps", "8", "--calibration-levels", "8", "--seq-len", "16", "--repeats", "1"])
    assert d["acceptance"]["passed"] and d["metrics"]["exact_logits_relative_l2"] < 1e-4 and d["structure"]["decoder_layers"] == 2
    d = _json_line([str(ROOT / "benchmark" / "snn_llm_gpt2_conversion.py"), "--device", "cpu", "--hidden", "32", "--heads", "2", "--vocab", "200",
                    "--max-length", "24", "--prefill-length", "8", "--max-samples", "2"])
    assert d["acceptance"]["passed"] and d["cache"]["equivalent"] and d["mlp"]["if_vs_qcfs_max_abs_error"] <= 1e-5


def test_distributed_precision_smoke_two_gloo_ranks():
    import os
    env = {**os.environ, "OMP_NUM_THREADS": "2"}
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nproc-per-node", "2", "--master-addr", "127.0.0.1", "--master-port", "29573",
                        str(ROOT / "benchmark" / "snn_llm_distributed_precision_smoke.py"), "--device", "cpu", "--precisions", "fp32", "bf16",
                        "--steps", "12", "--dim", "32", "--seq-len", "16"], capture_output=True, text=True, timeout=900, env=env)
    assert r.returncode == 0, r.stderr[-2000:]
    rows = [json.loads(line) for line in r.stdout.splitlines() if line.startswith("{")]
    assert [x["precision"] for x in rows] == ["fp32", "bf16"] and all(x["passed"] and x["ranks_identical"] for x in rows)
