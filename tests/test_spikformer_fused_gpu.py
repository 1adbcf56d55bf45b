"""The fused channels-last Spikformer schedule.

Oracle: the same schedule written with plain PyTorch ops — fp32 BatchNorm / max-pool / eager LIF
rule on the bf16 tensors, rounding to bf16 at exactly the points where the fused kernels write
to memory.  Spikes must then agree almost everywhere and autograd of the oracle gives the
reference gradients.  The module-by-module path (which rounds at other points) is compared only
statistically."""
import pytest
import torch
import torch.nn.functional as F

from spikingjelly_b200.activation_based import functional, neuron
from spikingjelly_b200.models import spikformer

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF = torch.bfloat16


def _lif32(x32, lif):
    """Eager fp32 LIF over T for a fresh neuron; returns fp32 spikes."""
    ref = neuron.LIFNode(tau=lif.tau, decay_input=lif.decay_input, v_threshold=lif.v_threshold, v_reset=lif.v_reset,
                         surrogate_function=lif.surrogate_function, detach_reset=lif.detach_reset, step_mode="m")
    ref.train()
    return ref(x32)


def _bn32(y16, bn, dims):
    y = y16.float()
    mean = y.mean(dim=dims, keepdim=True)
    var = y.var(dim=dims, unbiased=False, keepdim=True)
    shape = [1] * y.dim()
    shape[-1] = -1
    return (y - mean) * torch.rsqrt(var + bn.eps) * bn.weight.view(shape) + bn.bias.view(shape)


def _oracle(net, x):
    """x: [B, 3, H, W] static image.  Mirrors models/_spikformer_fused.py op by op."""
    T = net.T
    B = x.shape[0]
    h = x.to(BF).contiguous(memory_format=torch.channels_last)
    stem = net.patch_embed
    for i, st in enumerate(stem.stages):
        conv, bn = st.conv_bn.block[0], st.conv_bn.block[1]
        y = F.conv2d(h, conv.weight.to(BF), None, 1, 1).permute(0, 2, 3, 1)            # NHWC bf16
        z = _bn32(y, bn, (0, 1, 2))
        p = F.max_pool2d(z.permute(0, 3, 1, 2), 3, 2, 1).permute(0, 2, 3, 1)           # fp32 NHWC
        seq = p.unsqueeze(0).expand(T, *p.shape) if i == 0 else p.reshape(T, B, *p.shape[1:])
        s = _lif32(seq, st.neuron).to(BF)                                              # [T, B, OH, OW, C]
        h = s.flatten(0, 1).permute(0, 3, 1, 2)
    pe = stem.positional_encoding
    conv, bn = pe.conv_bn.block[0], pe.conv_bn.block[1]
    y = F.conv2d(h, conv.weight.to(BF), None, 1, 1).permute(0, 2, 3, 1)
    n, hh, ww, C = y.shape
    rows = y.reshape(T, B * hh * ww, C)
    res = h.permute(0, 2, 3, 1).reshape(T, B * hh * ww, C)
    X = (_lif32(_bn32(rows, bn, (0, 1)), pe.neuron) + res.float()).to(BF)
    L = hh * ww
    M = T * B * L
    for blk in net.blocks:
        attn, mlp = blk.attn, blk.mlp
        Hh, d = attn.num_heads, C // attn.num_heads

        def lin(a16, conv1d):
            return (a16.reshape(M, -1) @ conv1d.weight.squeeze(-1).to(BF).t()).reshape(T, B * L, -1)
        S = _lif32(_bn32(lin(X, attn.qkv_conv_bn[0]), attn.qkv_conv_bn[1], (0, 1)), attn.qkv_lif).to(BF)
        q, k, v = S.float().view(T, B, L, 3, Hh, d).unbind(3)
        kv = torch.einsum("tblhd,tblhe->tbhde", k, v).to(BF).float()        # the kernel keeps K^T V in bf16
        a = (torch.einsum("tblhd,tbhde->tblhe", q, kv) * attn.scale).reshape(T, B * L, C).to(BF)
        A = _lif32(a.float(), attn.attn_lif).to(BF)
        X1 = (_lif32(_bn32(lin(A, attn.proj_conv_bn[0]), attn.proj_conv_bn[1], (0, 1)), attn.proj_lif) + X.float()).to(BF)
        F1 = _lif32(_bn32(lin(X1, mlp.fc1[0]), mlp.fc1[1], (0, 1)), mlp.neuron1).to(BF)
        X = (_lif32(_bn32(lin(F1, mlp.fc2[0]), mlp.fc2[1], (0, 1)), mlp.neuron2) + X1.float()).to(BF)
    feat = X.view(T, B, L, C).mean(dim=2)
    return F.linear(feat, net.head.weight.to(BF), net.head.bias.to(BF))


def _grads(net):
    return {n: p.grad.detach().float().clone() for n, p in net.named_parameters() if p.grad is not None}


def _make(depths=2, dims=128, heads=4, T=4, size=64, classes=16):
    torch.manual_seed(0)
    return spikformer.Spikformer(T=T, img_size_h=size, img_size_w=size, embed_dims=dims, num_heads=heads, depths=depths,
                                 num_classes=classes, backend="cuda").to(DEV)


@pytest.mark.parametrize("dims,heads", [(128, 4), (128, 2)])     # head_dim 32 and 64
def test_fused_matches_same_schedule_oracle(dims, heads):
    net = _make(dims=dims, heads=heads)
    x = torch.randn(8, 3, 64, 64, device=DEV)
    y = torch.randint(0, 16, (8,), device=DEV)
    net.zero_grad(set_to_none=True)
    out_o = _oracle(net, x)
    F.cross_entropy(out_o.float().mean(0), y).backward()
    g_o = _grads(net)
    net.zero_grad(set_to_none=True)
    with torch.autocast("cuda", dtype=BF):
        out_f = net(x)
    F.cross_entropy(out_f.float().mean(0), y).backward()
    functional.reset_net(net)
    g_f = _grads(net)
    from spikingjelly_b200.ops import gemm
    gemm.check_status(x)
    cos = F.cosine_similarity(out_f.float().flatten(), out_o.float().flatten(), dim=0).item()
    assert cos > 0.9999, cos                     # measured 0.9999998
    worst = min((F.cosine_similarity(g_f[n].flatten(), g_o[n].flatten(), dim=0).item(), n)
                for n in g_o if g_o[n].norm() > 0)
    assert worst[0] > 0.999, worst                # measured 0.99992 (batch-norm affine parameters of the stem)


def test_fused_vs_modular_statistics():
    net = _make()
    x = torch.randn(8, 3, 64, 64, device=DEV)
    outs = []
    for fused in (False, True):
        net.fused = fused
        with torch.no_grad(), torch.autocast("cuda", dtype=BF):
            outs.append(net(x).float())
        functional.reset_net(net)
    assert outs[0].shape == outs[1].shape
    assert F.cosine_similarity(outs[0].flatten(), outs[1].flatten(), dim=0) > 0.8
    assert abs(outs[0].std() - outs[1].std()) < 0.2 * outs[0].std()


def test_sequence_input_and_eval_mode():
    net = _make(depths=1, dims=64, heads=2, T=2, size=32, classes=4)
    x = torch.randn(2, 4, 3, 32, 32, device=DEV)
    for m in net.modules():
        if isinstance(m, torch.nn.modules.batchnorm._BatchNorm):
            m.momentum = 1.0      # running statistics = statistics of this batch, so eval mode stays active
    with torch.autocast("cuda", dtype=BF):
        out = net(x)
    out.float().sum().backward()
    functional.reset_net(net)
    bn = net.blocks[0].mlp.fc1[1]
    assert int(bn.num_batches_tracked) == 1 and not torch.allclose(bn.running_mean, torch.zeros_like(bn.running_mean))
    net.eval()
    with torch.no_grad(), torch.autocast("cuda", dtype=BF):
        a = net(x).float()
        functional.reset_net(net)
        net.fused = False
        b = net(x).float()
    assert a.abs().sum() > 0
    assert F.cosine_similarity(a.flatten(), b.flatten(), dim=0) > 0.9


def _reference_spikformer(**cfg):
    """The unmodified reference package's Spikformer (installed under ``baseline/_ref``), or a skip."""
    import sys
    from pathlib import Path
    ref = Path(__file__).resolve().parents[1] / "baseline" / "_ref"
    if not (ref / "spikingjelly").is_dir():
        pytest.skip("reference package is not installed under baseline/_ref")
    if str(ref) not in sys.path:
        sys.path.insert(0, str(ref))
    from spikingjelly.activation_based import functional as ref_functional
    from spikingjelly.activation_based.model import spikformer as ref_spikformer
    return ref_spikformer.Spikformer(backend="torch", **cfg), ref_functional


def test_against_the_reference_package_with_shared_weights():
    cfg = dict(T=4, img_size_h=64, img_size_w=64, embed_dims=128, num_heads=4, depths=2, num_classes=16)
    ref, ref_functional = _reference_spikformer(**cfg)
    ref = ref.to(DEV)
    torch.manual_seed(0)
    net = spikformer.Spikformer(backend="cuda", **cfg).to(DEV)
    missing = net.load_state_dict(ref.state_dict(), strict=True)          # same module tree, same keys
    assert not missing.missing_keys and not missing.unexpected_keys
    x = torch.randn(8, 3, 64, 64, device=DEV)
    y = torch.randint(0, 16, (8,), device=DEV)
    # 1. fp32, module by module: the same arithmetic as the reference's eager path
    net.fused = False
    out_r = ref(x)
    F.cross_entropy(out_r.mean(0), y).backward()
    ref_functional.reset_net(ref)
    out_m = net(x)
    F.cross_entropy(out_m.mean(0), y).backward()
    functional.reset_net(net)
    g_r = {n: p.grad.detach().clone() for n, p in ref.named_parameters() if p.grad is not None}
    g_m = _grads(net)
    assert torch.allclose(out_m, out_r, rtol=1e-3, atol=1e-4), (out_m - out_r).abs().max()
    for n in g_r:
        if g_r[n].norm() > 0:
            assert F.cosine_similarity(g_m[n].flatten(), g_r[n].flatten(), dim=0) > 0.999, n
    # 2. the fused bf16 schedule against the reference.  A randomly initialised spiking network amplifies rounding: the
    #    reference's own bf16-autocast output has cosine 0.93 with its fp32 output.  The fused schedule must agree with
    #    the fp32 reference at least as well as the reference's bf16 run does (gradients of this chaotic pair are not
    #    comparable parameter by parameter; test_fused_matches_same_schedule_oracle checks them to 0.999).
    net.zero_grad(set_to_none=True)
    net.fused = True
    with torch.autocast("cuda", dtype=BF):
        out_f = net(x)
        out_r16 = ref(x)
    ref_functional.reset_net(ref)
    loss_f = F.cross_entropy(out_f.float().mean(0), y)
    loss_f.backward()
    functional.reset_net(net)
    agree = lambda a, b: F.cosine_similarity(a.float().flatten(), b.float().flatten(), dim=0).item()
    assert agree(out_f, out_r) > agree(out_r16, out_r) - 0.03, (agree(out_f, out_r), agree(out_r16, out_r))
    assert agree(out_f.float().mean(0), out_r.mean(0)) > 0.95
    assert abs(float(loss_f) - float(F.cross_entropy(out_r.detach().mean(0), y))) < 0.05
    assert all(torch.isfinite(g).all() for g in _grads(net).values())
