"""SpikeZIP-TF conversion: the time-summed output of the converted network equals the quantised ANN."""
import pytest
import torch
import torch.nn as nn

from spikingjelly_b200.activation_based import functional
from spikingjelly_b200.activation_based.ann2snn import ModuleConverter
from spikingjelly_b200.activation_based.ann2snn.recipes import SpikeZIPTFQANNRecipe
from spikingjelly_b200.activation_based.ann2snn.recipes import spikezip_qann as Z


class Quan(nn.Module):
    """LSQ-style activation quantiser: ``clamp(round(x / s), neg_min, pos_max) * s``."""

    def __init__(self, s: float, level: int, sym: bool):
        super().__init__()
        self.s = nn.Parameter(torch.tensor(float(s)))
        self.level, self.sym = level, sym
        self.pos_max = torch.tensor(float(level // 2 - 1 if sym else level - 1))
        self.neg_min = torch.tensor(float(-level // 2 if sym else 0))

    def forward(self, x):
        return torch.clamp(torch.floor(x / self.s + 0.5), float(self.neg_min), float(self.pos_max)) * self.s


class QAttention(nn.Module):
    def __init__(self, dim, heads, level):
        super().__init__()
        self.num_heads, self.scale = heads, (dim // heads) ** -0.5
        self.qkv = nn.Linear(dim, 3 * dim)
        self.quan_q, self.quan_k, self.quan_v = Quan(0.25, level, True), Quan(0.25, level, True), Quan(0.25, level, True)
        self.attn_quan = Quan(1.0 / (level - 1), level, False)
        self.after_attn_quan = Quan(0.125, level, True)
        self.proj = nn.Linear(dim, dim)
        self.quan_proj = Quan(0.125, level, True)

    def forward(self, x):
        b, l, c = x.shape
        q, k, v = self.qkv(x).chunk(3, dim=-1)
        split = lambda t: t.view(b, l, self.num_heads, c // self.num_heads).transpose(1, 2)   # noqa: E731
        q, k, v = split(self.quan_q(q)), split(self.quan_k(k)), split(self.quan_v(v))
        p = self.attn_quan(torch.softmax(q @ k.transpose(-1, -2) * self.scale, dim=-1))
        ctx = self.after_attn_quan(p @ v).transpose(1, 2).reshape(b, l, c)
        return self.quan_proj(self.proj(ctx))


class QMLP(nn.Module):
    def __init__(self, level=16):
        super().__init__()
        self.inq = Quan(0.125, level, True)
        self.fc1, self.relu, self.q1 = nn.Linear(12, 24), nn.ReLU(), Quan(0.1, level, False)
        self.fc2, self.q2 = nn.Linear(24, 8), Quan(0.2, level, True)

    def forward(self, x):
        return self.q2(self.fc2(self.q1(self.relu(self.fc1(self.inq(x))))))


def _run(snn, x, T):
    functional.reset_net(snn)
    total = 0
    with torch.no_grad():
        for t in range(T):
            total = total + snn(x if t == 0 else torch.zeros_like(x))
    return total


def test_mlp_equals_quantised_ann():
    torch.manual_seed(0)
    qann = QMLP().eval()
    x = torch.randn(5, 12)
    snn = ModuleConverter(SpikeZIPTFQANNRecipe(time_steps=64, model_family="generic")).convert(qann)
    assert isinstance(snn.fc1, Z.SpikeZIPLinear) and isinstance(snn.relu, nn.Identity) and snn.time_steps == 64
    from spikingjelly_b200.activation_based.neuron import STBIFNeuron
    assert isinstance(snn.q1, STBIFNeuron) and snn.q1.level == 16
    with torch.no_grad():
        want = qann(x)
    torch.testing.assert_close(_run(snn, x, 64), want, rtol=0, atol=1e-5)
    torch.testing.assert_close(_run(snn, x, 64), want, rtol=0, atol=1e-5)          # reset_net restores the start state


def test_attention_and_layernorm_block_converges_to_quantised_ann():
    torch.manual_seed(1)

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.inq = Quan(0.125, 32, True)
            self.norm = nn.LayerNorm(16)
            self.nq = Quan(0.125, 32, True)
            self.attn = QAttention(16, 2, 32)

        def forward(self, x):
            return self.attn(self.nq(self.norm(self.inq(x))))

    qann = Block().eval()
    snn = ModuleConverter(SpikeZIPTFQANNRecipe(time_steps=128, model_family="vit")).convert(qann)
    assert isinstance(snn.attn, Z.SpikeZIPSelfAttention) and isinstance(snn.norm, Z.SpikeZIPLayerNorm)
    x = torch.randn(2, 6, 16)
    with torch.no_grad():
        want = qann(x)
    got = _run(snn, x, 128)
    # every output is a multiple of the last quantiser's step; at most a few land one step off (ties at the rounding point)
    off = ((got - want).abs() > 1e-5).float().mean().item()
    assert off <= 0.05 and (got - want).abs().max().item() <= 0.125 + 1e-5


def test_embedding_and_validation():
    emb = Z.SpikeZIPEmbedding(nn.Embedding(10, 4))
    ids = torch.tensor([[1, 2, 3]])
    first, second = emb(ids), emb(ids)
    assert first.abs().sum() > 0 and second.abs().sum() == 0
    with pytest.raises(ValueError):
        ModuleConverter(SpikeZIPTFQANNRecipe(time_steps=0)).convert(nn.Linear(2, 2))
    with pytest.raises(ValueError):
        ModuleConverter(SpikeZIPTFQANNRecipe(model_family="bert")).convert(nn.Linear(2, 2))


def _sequence_run(snn, x, T):
    functional.reset_net(snn)
    functional.set_step_mode(snn, "m")
    seq = torch.zeros(T, *x.shape)
    seq[0] = x
    with torch.no_grad():
        out = snn(seq)
    functional.set_step_mode(snn, "s")
    return out


def test_multi_step_mode_equals_the_single_step_loop():
    torch.manual_seed(2)

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.inq = Quan(0.125, 32, True)
            self.norm = nn.LayerNorm(16)
            self.nq = Quan(0.125, 32, True)
            self.attn = QAttention(16, 2, 32)
            self.fc, self.fq = nn.Linear(16, 8), Quan(0.1, 32, True)

        def forward(self, x):
            return self.fq(self.fc(self.attn(self.nq(self.norm(self.inq(x))))))

    snn = ModuleConverter(SpikeZIPTFQANNRecipe(time_steps=48, model_family="vit")).convert(Block().eval())
    x = torch.randn(2, 6, 16)
    functional.reset_net(snn)
    with torch.no_grad():
        loop = torch.stack([snn(x if t == 0 else torch.zeros_like(x)) for t in range(48)])
    seq = _sequence_run(snn, x, 48)
    torch.testing.assert_close(seq, loop, rtol=0, atol=1e-5)
    # a sequence split into two calls continues from the stored sums
    functional.reset_net(snn)
    functional.set_step_mode(snn, "m")
    full = torch.zeros(48, *x.shape)
    full[0] = x
    with torch.no_grad():
        halves = torch.cat([snn(full[:20]), snn(full[20:])])
    torch.testing.assert_close(halves, loop, rtol=0, atol=1e-5)


class _PatchEmbed(nn.Module):
    def __init__(self, dim, level):
        super().__init__()
        self.proj = nn.Sequential(nn.Conv2d(3, dim, 4, stride=4), Quan(0.125, level, True))

    def forward(self, x):
        return self.proj(x)


class _QBlock(nn.Module):
    def __init__(self, dim, level):
        super().__init__()
        self.norm1 = nn.Sequential(nn.LayerNorm(dim), Quan(0.125, level, True))
        self.attn = QAttention(dim, 2, level)

    def forward(self, x):
        return x + self.attn(self.norm1(x))


class TinyQViT(nn.Module):
    def __init__(self, dim=16, level=32):
        super().__init__()
        self.patch_embed = _PatchEmbed(dim, level)
        self.cls_token = nn.Parameter(torch.randn(1, 1, dim) * 0.1)
        self.pos_embed = nn.Parameter(torch.randn(1, 5, dim) * 0.1)
        self.blocks = nn.Sequential(_QBlock(dim, level))
        self.norm = nn.Sequential(nn.LayerNorm(dim), Quan(0.125, level, True))
        self.head = nn.Linear(dim, 7)

    def forward(self, x):
        x = self.patch_embed(x).flatten(2).transpose(1, 2)
        x = torch.cat((self.cls_token.expand(x.shape[0], -1, -1), x), dim=1) + self.pos_embed
        return self.head(self.norm(self.blocks(x))[:, 0])


def test_vit_class_token_and_position_embedding_enter_once():
    torch.manual_seed(3)
    qann = TinyQViT().eval()
    snn = ModuleConverter(SpikeZIPTFQANNRecipe(time_steps=64, model_family="vit")).convert(qann)
    x = torch.randn(2, 3, 8, 8)
    with torch.no_grad():
        want = qann(x)
    got = _run(snn, x, 64)
    assert ((got - want).abs() > 1e-4).float().mean().item() <= 0.05 and (got - want).abs().max().item() <= 0.2
    assert (_run(snn, x, 64) - got).abs().max().item() == 0          # reset_net restarts the step clock
    seq = _sequence_run(snn, x, 64).sum(0)
    torch.testing.assert_close(seq, got, rtol=0, atol=1e-5)
