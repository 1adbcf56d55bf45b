"""Training through the fused tensor-parallel path (``parallel/fused_tp_train.py``).

One GPU: the token-sharded model with one rank against the plain SNN-LLM on the same weights (loss and gradients agree up
to 16-bit rounding and the spikes it flips).  Two GPUs: each rank runs the two-rank model and, on a one-rank group of its
own, the same model unsharded; loss shares add up to the full loss, sliced weight gradients equal the matching slices and
replicated gradients add up to the full gradients."""
import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _cos(a, b):
    a, b = a.float().flatten(), b.float().flatten()
    if float(a.norm()) == 0.0 and float(b.norm()) == 0.0:
        return 1.0                              # a silent neuron layer: both gradients vanish
    return float(torch.dot(a, b) / (a.norm() * b.norm() + 1e-20))


def _tiny(dev, seed=0):
    from spikingjelly_b200.models import snn_llm
    torch.manual_seed(seed)
    # d_model / ranks and d_ffn / ranks stay multiples of 256 for two ranks; 2 x 128 tokens = 128 per rank
    model = snn_llm.snn_llm_tiny(vocab_size=512, d_model=512, n_layers=2, n_heads=8, d_ffn=1024, T=2, max_seq_len=128, backend="cuda").to(dev)
    with torch.no_grad():                       # larger weights than the default init, so that the neurons actually fire
        for p in model.parameters():
            if p.dim() == 2:
                p.mul_(6.0)
    return model


def test_one_rank_matches_the_plain_model():
    from spikingjelly_b200.parallel.fused_tp_train import FusedTPSNNLLM
    dev = torch.device("cuda")
    model = _tiny(dev)
    fused = FusedTPSNNLLM(model, batch=2, seq_len=128)
    tok = torch.randint(0, 512, (2, 128), device=dev, generator=torch.Generator(dev).manual_seed(1))
    with torch.autocast("cuda", dtype=torch.bfloat16):
        _, ref_loss = model(tok, labels=tok)
    ref_loss.backward()
    _, loss = fused(tok, labels=tok)
    loss.backward()
    fused.check()
    assert abs(float(loss) - float(ref_loss)) < 0.05 * abs(float(ref_loss)), (float(loss), float(ref_loss))
    pairs = [(fused.layers[0].w_in, model.blocks[0].attn.qkv.weight), (fused.layers[0].w_out, model.blocks[0].attn.proj.weight),
             (fused.layers[1].w_in, model.blocks[0].ffn.up.weight), (fused.layers[1].w_out, model.blocks[0].ffn.down.weight),
             (fused.layers[3].w_out, model.blocks[1].ffn.down.weight), (fused.layers[1].norm_weight, model.blocks[0].norm2.weight)]
    for ours, theirs in pairs:
        assert ours.grad is not None and ours.grad.shape == theirs.grad.shape
        assert _cos(ours.grad, theirs.grad) > 0.9, _cos(ours.grad, theirs.grad)
    assert _cos(model.lm_head.weight.grad, model.lm_head.weight.grad) > 0.99


def _worker(rank, world, init_file, out_dir):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", init_method=f"file://{init_file}", rank=rank, world_size=world, device_id=dev)
    solo_groups = [dist.new_group([r]) for r in range(world)]
    from spikingjelly_b200.parallel.fused_tp_train import FusedTPSNNLLM
    tok = torch.randint(0, 512, (2, 128), device=dev, generator=torch.Generator(dev).manual_seed(1))
    full = FusedTPSNNLLM(_tiny(dev), batch=2, seq_len=128, group=solo_groups[rank])
    _, full_loss = full(tok, labels=tok)
    full_loss.backward()
    torch.cuda.synchronize()
    dist.barrier()
    shard = FusedTPSNNLLM(_tiny(dev), batch=2, seq_len=128, timeout_s=20.0)
    _, share = shard(tok, labels=tok)
    share.backward()
    shard.check()
    total = share.detach().clone()
    dist.all_reduce(total)
    res = {"loss_full": float(full_loss), "loss_sum": float(total)}
    for i, (a, b) in enumerate(zip(shard.layers, full.layers)):
        rows, cols = a.w_in.shape[0], a.w_out.shape[1]
        res[f"w_in_{i}"] = _cos(a.w_in.grad, b.w_in.grad[rank * rows:(rank + 1) * rows])
        res[f"w_out_{i}"] = _cos(a.w_out.grad, b.w_out.grad[:, rank * cols:(rank + 1) * cols])
        g = a.norm_weight.grad.clone()
        dist.all_reduce(g)
        res[f"norm_{i}"] = _cos(g, b.norm_weight.grad)
    g = shard.lm_head.weight.grad.clone()
    dist.all_reduce(g)
    res["lm_head"] = _cos(g, full.lm_head.weight.grad)
    g = shard.embed.weight.grad.clone()
    dist.all_reduce(g)
    res["embed"] = _cos(g, full.embed.weight.grad)
    torch.save(res, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_ranks_match_the_unsharded_model():
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_worker, args=(2, os.path.join(d, "init"), d), nprocs=2, join=True)
        results = [torch.load(os.path.join(d, f"r{r}.pt")) for r in range(2)]
    for res in results:
        assert abs(res["loss_sum"] - res["loss_full"]) < 0.02 * abs(res["loss_full"]), res
        low = {k: v for k, v in res.items() if not k.startswith("loss") and v < 0.97}
        assert not low, low
