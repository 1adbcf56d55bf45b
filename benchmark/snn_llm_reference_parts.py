"""The SNN-LLM of ``models/snn_llm.py`` assembled from the REFERENCE package's public parts, for the reference arm of
``benchmark_snn_llm.py``: ``spikingjelly.activation_based.layer.Linear``, ``neuron.LIFNode(step_mode="m", backend="triton")``
(falls back to ``"torch"`` where Triton cannot run), the reference's DTensor tensor parallelism
(``distributed.tensor_parallel.parallelize_snn_module``: QKV / up column-wise with local output, O / down row-wise) and
plain PyTorch for what the reference has no module for (RMSNorm, rotary embedding, causal attention).  Nothing of this
framework is imported here; the reference itself has no model of this shape, so this is the baseline the task names:
the same architecture built by a user of the reference."""
import math
import sys
from pathlib import Path

import torch
import torch.nn as nn
import torch.nn.functional as F

REF_DIR = Path(__file__).resolve().parents[1] / "baseline" / "_ref"


def import_reference():
    if not (REF_DIR / "spikingjelly").exists():
        raise FileNotFoundError("baseline/_ref is empty: the reference is not installed")
    if str(REF_DIR) not in sys.path:
        sys.path.insert(0, str(REF_DIR))
    from spikingjelly.activation_based import functional, layer, neuron, surrogate
    return functional, layer, neuron, surrogate


def pick_backend(device) -> str:
    _, _, neuron, _ = import_reference()
    try:
        probe = neuron.LIFNode(step_mode="m", backend="triton").to(device)
        x = torch.randn(4, 1024, device=device, dtype=torch.bfloat16, requires_grad=True)
        probe(x).sum().backward()
        torch.cuda.synchronize()
        return "triton"
    except Exception as exc:
        sys.stderr.write(f"[reference parts] triton neuron backend unavailable ({type(exc).__name__}: {exc}); using torch\n")
        return "torch"


def build(n_layers: int, seq_len: int, backend: str, d_model=2048, n_heads=16, d_ffn=5504, vocab=32000, T=4, tau=2.0, eps=1e-6):
    functional, layer, neuron, surrogate = import_reference()
    head_dim = d_model // n_heads

    def lif():
        return neuron.LIFNode(tau=tau, detach_reset=True, surrogate_function=surrogate.ATan(), step_mode="m", backend=backend)

    class RMSNorm(nn.Module):
        def __init__(self):
            super().__init__()
            self.weight = nn.Parameter(torch.ones(d_model))

        def forward(self, x):
            out_dtype = torch.get_autocast_dtype("cuda") if (x.is_cuda and torch.is_autocast_enabled("cuda")) else x.dtype
            with torch.autocast("cuda", enabled=False):
                return F.rms_norm(x.float(), (d_model,), self.weight.float(), eps).to(out_dtype)

    class Rope(nn.Module):
        def __init__(self):
            super().__init__()
            inv = 1.0 / (10000.0 ** (torch.arange(0, head_dim, 2).float() / head_dim))
            ang = torch.outer(torch.arange(seq_len).float(), inv)
            self.register_buffer("cos", torch.cat([ang.cos(), ang.cos()], -1), persistent=False)
            self.register_buffer("sin", torch.cat([ang.sin(), ang.sin()], -1), persistent=False)

        def forward(self, x):
            S, half = x.shape[-2], x.shape[-1] // 2
            rot = torch.cat([-x[..., half:], x[..., :half]], -1)
            return x * self.cos[:S].to(x.dtype) + rot * self.sin[:S].to(x.dtype)

    class Attention(nn.Module):
        def __init__(self):
            super().__init__()
            self.local_heads = n_heads
            self.qkv = layer.Linear(d_model, 3 * d_model, bias=False, step_mode="m")
            self.attn_lif = lif()
            self.proj = layer.Linear(d_model, d_model, bias=False, step_mode="m")
            self.rope = Rope()

        def forward(self, s):
            T_, B, S, _ = s.shape
            H = self.local_heads
            qkv = self.qkv(s).reshape(T_ * B, S, H, 3, head_dim)
            q, k, v = (qkv[:, :, :, i].transpose(1, 2) for i in range(3))
            a = F.scaled_dot_product_attention(self.rope(q), self.rope(k), v, is_causal=True)
            return self.proj(self.attn_lif(a.transpose(1, 2).reshape(T_, B, S, H * head_dim)))

    class FFN(nn.Module):
        def __init__(self):
            super().__init__()
            self.up = layer.Linear(d_model, d_ffn, bias=False, step_mode="m")
            self.lif = lif()
            self.down = layer.Linear(d_ffn, d_model, bias=False, step_mode="m")

        def forward(self, s):
            return self.down(self.lif(self.up(s)))

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.norm1, self.lif1, self.attn = RMSNorm(), lif(), Attention()
            self.norm2, self.lif2, self.ffn = RMSNorm(), lif(), FFN()

        def forward(self, h):
            h = h + self.attn(self.lif1(self.norm1(h)))
            return h + self.ffn(self.lif2(self.norm2(h)))

    class Model(nn.Module):
        def __init__(self):
            super().__init__()
            self.embed = nn.Embedding(vocab, d_model)
            self.blocks = nn.ModuleList(Block() for _ in range(n_layers))
            self.norm_f = RMSNorm()
            self.lm_head = nn.Linear(d_model, vocab, bias=False)
            for m in self.modules():
                if isinstance(m, (nn.Linear, nn.Embedding)):
                    nn.init.normal_(m.weight, 0.0, 0.02)
            for name, p in self.named_parameters():
                if name.endswith("proj.weight") or name.endswith("down.weight"):
                    nn.init.normal_(p, 0.0, 0.02 / math.sqrt(2 * n_layers))

        def forward(self, tokens, labels):
            functional.reset_net(self)
            x = self.embed(tokens)
            h = x.unsqueeze(0).expand(T, *x.shape)
            for blk in self.blocks:
                h = blk(h)
            logits = self.lm_head(self.norm_f(h.mean(0)))
            loss = F.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]).float(), labels[:, 1:].reshape(-1))
            return logits, loss

        def flops_per_token(self, seq):
            per_layer = 2 * (4 * d_model * d_model + 2 * d_model * d_ffn) + 4 * seq * d_model / 2
            return T * n_layers * per_layer + 2 * d_model * vocab

    return Model()


def tensor_parallel(model, world: int, device_type: str = "cuda"):
    """The reference's DTensor tensor parallelism over all ranks: QKV and up column-wise (outputs stay local shards, i.e.
    whole heads / FFN columns), O and down row-wise."""
    import_reference()
    from spikingjelly.activation_based.distributed.mesh import build_device_mesh
    from spikingjelly.activation_based.distributed.tensor_parallel.linear import parallelize_snn_module
    mesh = build_device_mesh(device_type, (world,), None)
    plan = {}
    for i, blk in enumerate(model.blocks):
        blk.attn.local_heads //= world
        plan[f"blocks.{i}.attn.qkv"] = "colwise_local_output"
        plan[f"blocks.{i}.attn.proj"] = "rowwise"
        plan[f"blocks.{i}.ffn.up"] = "colwise_local_output"
        plan[f"blocks.{i}.ffn.down"] = "rowwise"
    return parallelize_snn_module(model, mesh, plan, 0)
