"""Precision policies: configuration, capability checks, fallback, module conversion, reports."""
import json
import warnings

import pytest
import torch
import torch.nn as nn

from spikingjelly_b200.activation_based import functional, layer, neuron, precision
from spikingjelly_b200.activation_based.precision import capability


def _net():
    return nn.Sequential(layer.Linear(16, 32, step_mode="m"), neuron.LIFNode(step_mode="m"), layer.Conv1d(32, 32, 1, step_mode="m"),
                         nn.Sequential(nn.LayerNorm(32), nn.Linear(32, 64), nn.GELU(), nn.Linear(64, 32)),
                         nn.Sequential(nn.LayerNorm(32), nn.Linear(32, 16)), layer.Conv1d(16, 16, 3, padding=1, step_mode="m"))


def test_config_from_any():
    C = precision.PrecisionConfig
    assert C.from_any(None, "cpu") == C(device="cpu")
    assert C.from_any("BF16").mode == "bf16"
    assert C.from_any({"mode": "fp8", "device": torch.device("cuda", 0)}).device == "cuda:0"
    assert C.from_any(C("fp16"), "cuda:1").device == "cuda:1"
    with pytest.raises(TypeError):
        C.from_any(3)


def test_policy_resolution_and_descriptions():
    assert isinstance(precision.resolve_precision_policy("fp32"), precision.FP32Policy)
    bf = precision.resolve_precision_policy({"mode": "bf16", "device": "cpu"})
    assert bf.describe() == {"name": "bf16", "autocast": True, "device_type": "cpu", "dtype": "torch.bfloat16", "grad_scaler": False}
    assert bf.create_grad_scaler() is None
    for mode, cls in (("fp8", precision.Float8NativePolicy), ("fp8-torchao", precision.Float8TorchAOPolicy),
                      ("fp8-te", precision.Float8TransformerEnginePolicy)):
        p = precision.resolve_precision_policy(mode)
        assert isinstance(p, cls) and p.describe()["backend"] == "sjb200"
    with pytest.raises(ValueError, match="Unsupported precision mode"):
        precision.resolve_precision_policy("int4")


def test_capability_validation_rules():
    rep = precision.build_capability_report(nn.Linear(2, 2), "cpu", "fp16")
    with pytest.raises(RuntimeError, match="not supported on cpu"):
        precision.validate_capability(rep)
    precision.validate_capability(precision.build_capability_report(nn.Linear(2, 2), "cpu", "bf16"))
    rep = precision.build_capability_report(nn.Linear(2, 2), "cpu", "fp8")
    assert rep["can_convert"] and not rep["can_execute"] and rep["execution_note"] == "fp8 requires a CUDA device"
    with pytest.raises(RuntimeError, match="fp8 requires a CUDA device"):
        precision.validate_capability(rep)
    ok = dict(rep, native_fp8_available=True)
    precision.validate_capability(ok)
    with pytest.raises(RuntimeError, match="Unsupported precision mode"):
        precision.validate_capability(dict(rep, requested_mode="fp4"))


def test_fallback_to_fp32_and_strict_mode(tmp_path):
    net = _net()
    with pytest.warns(RuntimeWarning, match="falling back to fp32"):
        art = precision.prepare_model_for_precision(net, "cpu", "fp8")
    assert art.effective_config.mode == "fp32" and art.requested_config.mode == "fp8" and art.fallback_reason
    assert isinstance(art.policy, precision.FP32Policy) and art.model is net
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        precision.prepare_model_for_precision(net, "cpu", {"mode": "fp8", "strictness": "silent"})
    with pytest.raises(RuntimeError):
        precision.prepare_model_for_precision(net, "cpu", {"mode": "fp8", "strictness": "strict"})
    precision.save_precision_reports(art, str(tmp_path))
    runtime = json.loads((tmp_path / "precision_runtime.json").read_text())
    assert runtime["effective_config"]["mode"] == "fp32" and (tmp_path / "conversion_report.json").exists()
    rep = json.loads((tmp_path / "conversion_report.json").read_text())
    assert rep["convertible_linear"] == 1 and rep["convertible_torch_linear"] == 3 and rep["convertible_pointwise_conv1d"] == 1
    assert "5" in rep["unsupported_modules"] and "1" in rep["high_precision_modules"]


def test_bf16_training_step_on_cpu():
    torch.manual_seed(0)
    net = nn.Sequential(layer.Linear(8, 16), neuron.LIFNode(), layer.Linear(16, 4))
    art = precision.prepare_model_for_precision(net, "cpu", "bf16")
    opt = torch.optim.SGD(net.parameters(), lr=0.1)
    before = net[0].weight.detach().clone()
    with art.autocast_context():
        y = art.model(torch.rand(5, 8))
    assert y.dtype == torch.bfloat16
    norm = art.backward(y.float().pow(2).mean(), opt, clip_grad_norm=1.0)
    assert norm is not None and not torch.equal(before, net[0].weight)
    functional.reset_net(net)


@pytest.mark.parametrize("policy_cls", [precision.Float8NativePolicy, precision.Float8TransformerEnginePolicy])
def test_fp8_conversion_keeps_parameters_and_state_dict(policy_cls, monkeypatch):
    torch.manual_seed(0)
    net = _net()
    keys_before = list(net.state_dict().keys())
    params_before = {n: p for n, p in net.named_parameters()}
    x = torch.rand(3, 2, 16)
    functional.reset_net(net)
    policy = policy_cls(device_type="cpu")
    converted, report = precision.convert_model_for_precision(net, policy)
    assert list(converted.state_dict().keys()) == keys_before
    # linear layers keep their Parameter objects (the 1x1 convolution gets a re-shaped copy)
    assert all(any(p is q for q in converted.parameters()) for n, p in params_before.items() if not n.startswith("2."))
    assert isinstance(converted[0], precision.Float8LinearStepModule) and converted[0].step_mode == "m"
    assert isinstance(converted[2], precision.Float8PointwiseConv1dStepModule) and converted[2].weight.dim() == 3
    assert isinstance(converted[5], layer.Conv1d)                       # k=3 conv is left alone
    if policy_cls is precision.Float8TransformerEnginePolicy:
        assert isinstance(converted[3], precision.Float8TELayerNormMLPModule)
        assert isinstance(converted[4], precision.Float8TELayerNormLinearModule)
        assert {p["pattern"] for p in report.converted_patterns} == {"LayerNormMLP", "LayerNormLinear"}
    else:
        assert isinstance(converted[3][1], precision.Float8LinearStepModule)
    # round trip through a plain checkpoint of the unconverted architecture
    fresh = _net()
    fresh.load_state_dict(converted.state_dict())
    converted.load_state_dict(fresh.state_dict())
    # numerics on the host (emulated fp8): close to the fp32 network
    h = fresh[0](x); h = fresh[1](h); functional.reset_net(fresh)
    hq = converted[0](x)
    assert hq.shape == (3, 2, 32)
    assert torch.nn.functional.cosine_similarity(hq.flatten().float(), fresh[0](x).flatten(), dim=0) > 0.99


def test_attention_adapter_layouts():
    a = precision.TransformerEngineDotProductAttentionAdapter(2, 8, qkv_format="bshd", attn_mask_type="causal")
    q = torch.rand(3, 5, 2, 8)
    out = a(q, q, q)
    ref = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), q.transpose(1, 2), q.transpose(1, 2), is_causal=True)
    assert torch.allclose(out, ref.transpose(1, 2), atol=1e-6)
    with pytest.raises(ValueError):
        precision.TransformerEngineDotProductAttentionAdapter(2, 8, qkv_format="xyz")
