"""STA transformer recipe (role of the reference's ``test/activation_based/ann2snn`` STA cases): exactness of the
equivalent mode in both step modes on a ViT-shaped model with class token, position embedding, attention and MLP;
calibrated spike encoders; time constants; settings validation; the vmap lifting of tensor functions."""
import pytest
import torch
import torch.nn as nn

from spikingjelly_b200.activation_based import functional
from spikingjelly_b200.activation_based.ann2snn import Converter, STATransformerRecipe
from spikingjelly_b200.activation_based.ann2snn.recipes import sta_transformer as sta
from spikingjelly_b200.activation_based.ann2snn.recipes.step_mode_adapters import StepFunction


class Block(nn.Module):
    def __init__(self, d, heads):
        super().__init__()
        self.n1, self.n2 = nn.LayerNorm(d), nn.LayerNorm(d)
        self.attn = nn.MultiheadAttention(d, heads, batch_first=True)
        self.fc1, self.act, self.fc2 = nn.Linear(d, 2 * d), nn.GELU(), nn.Linear(2 * d, d)

    def forward(self, x):
        h = self.n1(x)
        x = x + self.attn(h, h, h, need_weights=False)[0]
        return x + self.fc2(self.act(self.fc1(self.n2(x))))


class TinyViT(nn.Module):
    def __init__(self, d=16, heads=2, patches=4, classes=5):
        super().__init__()
        self.embed = nn.Conv2d(3, d, 4, 4)
        self.cls_token = nn.Parameter(torch.randn(1, 1, d) * 0.5)
        self.pos_embed = nn.Parameter(torch.randn(1, patches + 1, d) * 0.5)
        self.blocks = nn.Sequential(Block(d, heads), Block(d, heads))
        self.norm, self.head = nn.LayerNorm(d), nn.Linear(d, classes)

    def forward(self, x):
        x = self.embed(x).flatten(2).transpose(1, 2)
        cls = self.cls_token.expand(x.shape[0], -1, -1)
        x = torch.cat((cls, x), dim=1) + self.pos_embed
        x = self.norm(self.blocks(x))
        return self.head(x[:, 0])


def _data(n=3):
    torch.manual_seed(0)
    return [torch.randn(2, 3, 8, 8) for _ in range(n)]


def test_equivalent_mode_is_exact_in_both_step_modes():
    torch.manual_seed(1)
    ann = TinyViT().eval()
    x = _data(1)[0]
    want = ann(x)
    T = 6
    snn = Converter(recipe=STATransformerRecipe(time_steps=T)).convert(ann)
    assert snn.time_steps == T
    assert any(isinstance(m, sta.STAConstant) for m in snn.modules()) and any(isinstance(m, StepFunction) for m in snn.modules())
    parts = torch.randn(T, *x.shape)
    parts = parts - parts.mean(0, keepdim=True) + x / T                     # any split of the input over time
    functional.set_step_mode(snn, "s")
    functional.reset_net(snn)
    got_s = sum(snn(parts[t]) for t in range(T))
    assert torch.allclose(got_s, want, atol=2e-4), (got_s - want).abs().max()
    functional.set_step_mode(snn, "m")
    functional.reset_net(snn)
    seq = snn(parts)
    assert seq.shape == (T, 2, 5)
    assert torch.allclose(seq.sum(0), want, atol=2e-4), (seq.sum(0) - want).abs().max()


def test_spiking_encoder_mode_calibrates_and_approaches_the_ann():
    torch.manual_seed(2)
    ann = TinyViT().eval()
    data = _data(4)
    T = 32
    recipe = STATransformerRecipe(dataloader=data, time_steps=T, mode="spiking_encoder", threshold_mode="mse", num_calibration_batches=3)
    snn = Converter(recipe=recipe).convert(ann)
    encoders = [m for m in snn.modules() if isinstance(m, sta.STASpikeEncoder)]
    # after every LayerNorm (5), GELU (2) and attention output (2)
    assert len(encoders) == 9 and all(bool((e.v_threshold > 0).all()) for e in encoders)
    x = data[0]
    functional.set_step_mode(snn, "m")
    functional.reset_net(snn)
    seq = torch.zeros(T, *x.shape)
    seq[0] = x
    out = snn(seq).sum(0)
    want = ann(x)
    cos = torch.nn.functional.cosine_similarity(out.flatten(), want.flatten(), dim=0)
    assert cos > 0.95, cos
    # every encoder output is a whole number of thresholds
    enc = encoders[0]
    functional.reset_net(snn)
    y = enc(torch.randn(T, 2, 5, 16))
    ratio = y / enc.v_threshold
    assert torch.allclose(ratio, ratio.round(), atol=1e-4)


def test_threshold_rules():
    a = torch.tensor([[1.0, -4.0], [2.0, 3.0]])
    assert torch.allclose(sta.sta_threshold(a, 4, mode="max"), torch.tensor([2.0, 4.0]) / 4)
    th = sta.sta_threshold(torch.randn(64, 8), 8, mode="mse")
    assert th.shape == (8,) and bool((th > 0).all())
    with pytest.raises(ValueError):
        sta.sta_threshold(torch.randn(4), 4)
    with pytest.raises(ValueError):
        sta.sta_threshold(a, 4, mode="median")


def test_time_constant_emits_once_per_reset():
    c = sta.STAConstant(torch.ones(1, 3), time_steps=4)
    assert c().sum() == 3 and c().sum() == 0
    functional.reset_net(c)
    c.step_mode = "m"
    seq = c()
    assert seq.shape == (4, 1, 3) and seq[0].sum() == 3 and seq[1:].sum() == 0
    assert c().sum() == 0


@pytest.mark.parametrize("kwargs,message", [
    ({"time_steps": 0}, "time_steps must be a positive integer"),
    ({"mode": "rate"}, "mode must be"),
    ({"threshold_mode": "median"}, "threshold_mode must be"),
    ({"threshold_scale": -1.0}, "threshold_scale must be positive"),
    ({"mode": "spiking_affine", "dataloader": [torch.zeros(1)]}, "supports only equivalent and spiking_encoder"),
    ({"spike_linear": True, "dataloader": [torch.zeros(1)]}, "supports only equivalent and spiking_encoder"),
    ({"mode": "spiking_encoder"}, "requires a dataloader"),
    ({"momentum": 1.5}, "momentum must be in"),
    ({"num_calibration_batches": 0}, "num_calibration_batches must be positive or None"),
    ({"eps": 0.0}, "eps must be a positive number"),
])
def test_settings_are_validated(kwargs, message):
    with pytest.raises(ValueError, match=message):
        Converter(recipe=STATransformerRecipe(**kwargs)).convert(TinyViT())


def test_attention_weights_cannot_be_used():
    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.attn = nn.MultiheadAttention(8, 2, batch_first=True)

        def forward(self, x):
            out, w = self.attn(x, x, x)
            return out + w.sum()
    with pytest.raises(ValueError, match="attention weights"):
        Converter(recipe=STATransformerRecipe(time_steps=2)).convert(Net())
