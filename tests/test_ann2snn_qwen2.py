"""Qwen2 conversion recipe on a tiny randomly initialised Hugging Face Qwen2 (grouped-query attention, left padding):
exact temporal-difference mode equals the source model, the spiking modes stay close, the KV cache path equals the full
pass, greedy generation runs, calibration survives a state-dict round trip, settings are validated."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from spikingjelly_b200.activation_based.ann2snn import ModuleConverter  # noqa: E402
from spikingjelly_b200.activation_based.ann2snn.recipes import qwen2 as Q  # noqa: E402


@pytest.fixture(scope="module")
def setup():
    cfg = transformers.Qwen2Config(vocab_size=97, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, max_position_embeddings=64, tie_word_embeddings=False)
    torch.manual_seed(0)
    model = transformers.Qwen2ForCausalLM(cfg).eval()
    ids = torch.randint(0, 97, (2, 9))
    mask = torch.ones_like(ids)
    mask[0, :3] = 0                                                  # left padding
    conf = Q.Qwen2SNNConfig(time_steps=8, calibration_levels=8)
    cal = Q.calibrate_qwen2_snn(model, [{"input_ids": ids, "attention_mask": mask}], conf)
    snn = ModuleConverter(Q.Qwen2SNNRecipe(cal, conf)).convert(model)
    return model, snn, ids, mask, cal, conf


def test_exact_mode_equals_the_source(setup):
    model, snn, ids, mask, _, _ = setup
    with torch.no_grad():
        want = model(input_ids=ids, attention_mask=mask).logits
        snn._reset_state()
        got = snn(ids, mask, encoding_mode="exact_td").logits
    assert torch.allclose(got[mask.bool()], want[mask.bool()], atol=1e-5)


@pytest.mark.parametrize("mode", ["signed_if", "qcfs_sg"])
def test_spiking_modes_stay_close(setup, mode):
    model, snn, ids, mask, _, _ = setup
    with torch.no_grad():
        want = model(input_ids=ids, attention_mask=mask).logits[mask.bool()]
        snn._reset_state()
        got = snn(ids, mask, encoding_mode=mode).logits[mask.bool()]
    assert torch.nn.functional.cosine_similarity(got.flatten(), want.flatten(), dim=0) > 0.98


def test_cache_continuation_equals_full_pass(setup):
    _, snn, ids, _, _, _ = setup
    x = ids[1:]
    with torch.no_grad():
        snn._reset_state()
        full = snn(x, encoding_mode="exact_td").logits
        snn._reset_state()
        first = snn(x[:, :6], torch.ones(1, 6, dtype=torch.long), encoding_mode="exact_td", use_cache=True)
        snn._reset_state()
        rest = snn(x[:, 6:], torch.ones(1, 9, dtype=torch.long), encoding_mode="exact_td", use_cache=True, past_key_values=first.past_key_values)
    assert rest.past_key_values.get_seq_length() == 9
    assert torch.allclose(rest.logits, full[:, 6:], atol=1e-5)
    summary = rest.past_key_values.storage_summary()
    assert summary["stored_cache_logical_bytes"] > 0 and summary["temporal_prefix_materialization_bytes"] == 0
    with pytest.raises(ValueError, match="use_cache=True"):
        snn(x[:, 6:], torch.ones(1, 9, dtype=torch.long), past_key_values=first.past_key_values)


def test_greedy_generation(setup):
    model, snn, ids, _, _, _ = setup
    out = snn.generate(ids[1:], max_new_tokens=3)
    assert out.shape == (1, 12) and torch.equal(out[:, :9], ids[1:])
    with pytest.raises(ValueError):
        snn.generate(ids[1:], max_new_tokens=1, do_sample=True)
    with pytest.raises(ValueError):
        snn.generate(ids[1:], max_new_tokens=-1)


def test_calibration_round_trip_and_summaries(setup, tmp_path):
    _, snn, _, _, cal, conf = setup
    torch.save(cal.state_dict(), tmp_path / "cal.pt")
    back = Q.Qwen2SNNCalibration.from_state_dict(torch.load(tmp_path / "cal.pt", weights_only=True))
    assert torch.equal(back.input_scale, cal.input_scale) and len(back.layer_scales) == 2
    assert all(torch.equal(back.layer_scales[1][n], cal.layer_scales[1][n]) for n in Q.SCALE_NAMES)
    assert back.valid_token_count == cal.valid_token_count == 15
    bad = cal.state_dict()
    bad["tensors"]["layer.0.extra"] = torch.ones(1)
    with pytest.raises(ValueError):
        Q.Qwen2SNNCalibration.from_state_dict(bad)
    s = snn.structure_summary()
    assert s["signed_encoders"] == 9 and s["decoder_layers"] == 2 and s["temporal_layout"] == "[T,B,S,H]"
    assert len(snn.encoder_statistics()) == 9
    other = Q.Qwen2SNNConfig(time_steps=16, calibration_levels=8)
    with pytest.raises(ValueError, match="time_steps does not match"):
        ModuleConverter(Q.Qwen2SNNRecipe(cal, other)).convert(setup[0])


def test_quantile_calibration_uses_a_bounded_reservoir(setup):
    model, _, ids, mask, _, _ = setup
    conf = Q.Qwen2SNNConfig(time_steps=8, calibration_levels=4, calibration_quantile=0.9, calibration_reservoir_size=7)
    cal = Q.calibrate_qwen2_snn(model, [{"input_ids": ids, "attention_mask": mask}] * 3, conf)
    assert cal.input_scale.shape == (32,) and bool((cal.input_scale > 0).all())
    assert cal.layer_scales[0]["mlp"].shape == (64,)


@pytest.mark.parametrize("kwargs,error", [({"time_steps": 0}, ValueError), ({"time_steps": 2.0}, TypeError),
                                          ({"calibration_levels": 64}, ValueError), ({"calibration_quantile": 0.0}, ValueError),
                                          ({"calibration_reservoir_size": 0}, ValueError), ({"neuron_backend": "cupy"}, ValueError)])
def test_config_validation(kwargs, error):
    with pytest.raises(error):
        Q.Qwen2SNNConfig(**kwargs)


def test_source_checks(setup):
    model = setup[0]
    model.train()
    try:
        with pytest.raises(ValueError, match="evaluation-mode"):
            Q.calibrate_qwen2_snn(model, [], setup[5])
    finally:
        model.eval()
    with pytest.raises(TypeError):
        Q.calibrate_qwen2_snn(torch.nn.Linear(2, 2), [], setup[5])
