"""The fused channels-last Spikformer schedule against the module-by-module path."""
import pytest
import torch
import torch.nn.functional as F

from spikingjelly_b200.activation_based import functional
from spikingjelly_b200.models import spikformer

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _step(net, x, y, fused):
    net.fused = fused
    net.zero_grad(set_to_none=True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out = net(x)
    loss = F.cross_entropy(out.float().mean(0), y)
    loss.backward()
    functional.reset_net(net)
    return out.detach().float(), loss.item(), {n: p.grad.detach().float().clone() for n, p in net.named_parameters()}


@pytest.mark.parametrize("static", [True, False])
def test_fused_matches_modular(static):
    torch.manual_seed(0)
    net = spikformer.Spikformer(T=4, img_size_h=64, img_size_w=64, embed_dims=128, num_heads=4, depths=2,
                                num_classes=16, backend="cuda").to(DEV)
    x = torch.randn(8, 3, 64, 64, device=DEV)
    if not static:
        x = x.unsqueeze(0).repeat(4, 1, 1, 1, 1) + 0.05 * torch.randn(4, 8, 3, 64, 64, device=DEV)
    y = torch.randint(0, 16, (8,), device=DEV)
    sd = {k: v.clone() for k, v in net.state_dict().items()}
    out_m, loss_m, g_m = _step(net, x, y, fused=False)
    net.load_state_dict(sd)
    out_f, loss_f, g_f = _step(net, x, y, fused=True)
    # bf16 pipelines with different rounding points: compare statistically
    assert out_f.shape == out_m.shape
    assert abs(loss_f - loss_m) < 0.05 * abs(loss_m) + 0.05
    cos = F.cosine_similarity(out_f.flatten(), out_m.flatten(), dim=0).item()
    assert cos > 0.98, cos
    for name in ("head.weight", "blocks.1.mlp.fc2.0.weight", "blocks.0.attn.qkv_conv_bn.0.weight",
                 "patch_embed.stages.3.conv_bn.block.0.weight", "patch_embed.stages.0.conv_bn.block.0.weight"):
        c = F.cosine_similarity(g_f[name].flatten(), g_m[name].flatten(), dim=0).item()
        assert c > 0.75, (name, c)     # spike flips from different rounding points decorrelate slowly
    from spikingjelly_b200.ops import gemm
    gemm.check_status(x)


def test_fused_eval_and_running_stats():
    torch.manual_seed(0)
    net = spikformer.Spikformer(T=2, img_size_h=32, img_size_w=32, embed_dims=64, num_heads=2, depths=1,
                                num_classes=4, backend="cuda").to(DEV)
    x = torch.randn(4, 3, 32, 32, device=DEV)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        net(x)
    functional.reset_net(net)
    bn = net.blocks[0].mlp.fc1[1]
    assert int(bn.num_batches_tracked) == 1 and not torch.allclose(bn.running_mean, torch.zeros_like(bn.running_mean))
    net.eval()
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        a = net(x).float()
        functional.reset_net(net)
        net.fused = False
        b = net(x).float()
    assert F.cosine_similarity(a.flatten(), b.flatten(), dim=0) > 0.98
