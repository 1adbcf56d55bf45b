"""SNN-LLM: shapes, causality, training step, and tensor-parallel equivalence on gloo ranks."""
import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from spikingjelly_b200.models import snn_llm as M


def test_shapes_causality_and_training_step():
    torch.manual_seed(0)
    net = M.snn_llm_tiny()
    tok = torch.randint(0, 256, (2, 16))
    logits, loss = net(tok, labels=tok)
    assert logits.shape == (2, 16, 256) and torch.isfinite(loss) and abs(loss.item() - 5.545) < 0.5      # ~ln(256)
    loss.backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in net.parameters())
    # a change of a later token must not change earlier logits
    tok2 = tok.clone()
    tok2[:, 10] = (tok2[:, 10] + 1) % 256
    with torch.no_grad():
        a, b = net(tok), net(tok2)
    assert torch.allclose(a[:, :10], b[:, :10], atol=1e-5) and not torch.allclose(a[:, 10:], b[:, 10:], atol=1e-5)
    # repeated calls are deterministic: the neuron states are reset at entry
    with torch.no_grad():
        assert torch.equal(net(tok), a)
    opt = torch.optim.AdamW(net.parameters(), lr=3e-3)
    first = None
    for _ in range(8):
        opt.zero_grad()
        _, loss = net(tok, labels=tok)
        loss.backward()
        opt.step()
        first = first if first is not None else loss.item()
    assert loss.item() < first


def test_benchmark_shape_parameter_count():
    cfg = M.SNNLLMConfig()
    per_layer = 4 * cfg.d_model ** 2 + 2 * cfg.d_model * cfg.d_ffn + 2 * cfg.d_model
    total = cfg.n_layers * per_layer + 2 * cfg.vocab_size * cfg.d_model + cfg.d_model
    assert 1.0e9 < total < 1.2e9 and cfg.head_dim == 128
    rope = M.RotaryEmbedding(8, 16)
    x = torch.randn(1, 2, 16, 8)
    y = rope(x)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5) and torch.allclose(y[..., 0, :], x[..., 0, :])
    # relative property: <rope(q)_i, rope(k)_j> depends on i - j only
    q, k = torch.randn(8), torch.randn(8)
    qq, kk = rope(q.expand(1, 1, 16, 8)), rope(k.expand(1, 1, 16, 8))
    assert torch.allclose((qq[0, 0, 5] * kk[0, 0, 3]).sum(), (qq[0, 0, 9] * kk[0, 0, 7]).sum(), atol=1e-4)


def _tp_worker(rank, world, init_file, out_dir):
    dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=world)
    torch.manual_seed(0)
    ref = M.snn_llm_tiny()
    torch.manual_seed(0)
    net = M.parallelize_snn_llm(M.snn_llm_tiny())
    tok = torch.randint(0, 256, (2, 12), generator=torch.Generator().manual_seed(1))
    lr, ll = ref(tok, labels=tok)
    ll.backward()
    ln, ls = net(tok, labels=tok)
    ls.backward()
    n = 128 // world
    res = {
        "logits": (ln - lr).abs().max().item(),
        "up": (net.blocks[0].ffn.up.weight.grad - ref.blocks[0].ffn.up.weight.grad[rank * n:(rank + 1) * n]).abs().max().item(),
        "down": (net.blocks[1].ffn.down.weight.grad - ref.blocks[1].ffn.down.weight.grad[:, rank * n:(rank + 1) * n]).abs().max().item(),
        "qkv": (net.blocks[0].attn.qkv.weight.grad - ref.blocks[0].attn.qkv.weight.grad[rank * 96:(rank + 1) * 96]).abs().max().item(),
        "norm": (net.blocks[0].norm1.weight.grad - ref.blocks[0].norm1.weight.grad).abs().max().item(),
        "embed": (net.embed.weight.grad - ref.embed.weight.grad).abs().max().item(),
    }
    torch.save(res, os.path.join(out_dir, f"r{rank}.pt"))
    dist.destroy_process_group()


def test_tensor_parallel_matches_unsharded():
    world = 2
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_tp_worker, args=(world, os.path.join(d, "init"), d), nprocs=world, join=True)
        for r in range(world):
            res = torch.load(os.path.join(d, f"r{r}.pt"))
            assert all(v < 2e-5 for v in res.values()), res


@pytest.mark.gpu
def test_native_backend_bf16_step_on_gpu():
    torch.manual_seed(0)
    net = M.snn_llm_tiny(backend="cuda", d_model=256, n_heads=4, d_ffn=512, T=4).cuda()
    tok = torch.randint(0, 256, (4, 64), device="cuda")
    with torch.autocast("cuda", dtype=torch.bfloat16):
        _, loss = net(tok, labels=tok)
    loss.backward()
    assert torch.isfinite(loss) and all(torch.isfinite(p.grad).all() for p in net.parameters())


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_fused_rope_qkv_matches_eager(dtype):
    from spikingjelly_b200 import ops
    from spikingjelly_b200.models.snn_llm import RotaryEmbedding
    from spikingjelly_b200.ops import rope as rope_ops
    ops.require()
    torch.manual_seed(0)
    N, S, H, D = 3, 37, 4, 64
    rope = RotaryEmbedding(D, 64).cuda()
    qkv = torch.randn(N, S, H, 3, D, device="cuda").to(dtype).requires_grad_(True)
    q, k, v = rope_ops.rope_qkv(qkv, rope.cos, rope.sin)
    ref = qkv.detach().float().requires_grad_(True)
    qr, kr, vr = (ref[:, :, :, i].transpose(1, 2) for i in range(3))            # [N, H, S, D]
    qr, kr = rope(qr), rope(kr)
    tol = dict(rtol=2e-2, atol=2e-2) if dtype is torch.bfloat16 else dict(rtol=3e-3, atol=3e-3)
    for a, b in ((q, qr), (k, kr), (v, vr)):
        assert a.shape == (N, S, H, D) and a.is_contiguous()
        torch.testing.assert_close(a.transpose(1, 2).float(), b, **tol)
    gq, gk, gv = (torch.randn(N, S, H, D, device="cuda").to(dtype) for _ in range(3))
    torch.autograd.backward([q, k, v], [gq, gk, gv])
    torch.autograd.backward([qr, kr, vr], [g.float().transpose(1, 2) for g in (gq, gk, gv)])
    torch.testing.assert_close(qkv.grad.float(), ref.grad, **tol)
