"""Spikformer: spiking vision transformer.

Stem: four ``Conv3x3 -> BN -> MaxPool(3, 2, 1) -> LIF`` stages (channels ``d/8, d/4, d/2, d``,
total stride 16) and a ``Conv3x3 -> BN -> LIF`` positional branch added residually.
Encoder block: ``x + SSA(x)`` then ``x + MLP(x)`` on tokens ``[T, N, C, L]``.
Head: mean over tokens, ``Linear``.  Output ``[T, N, num_classes]``.

Module names are chosen so that ``state_dict`` keys equal the reference's:
``patch_embed.stages.{i}.conv_bn.block.{0,1}.*``, ``patch_embed.positional_encoding.conv_bn.block.*``,
``blocks.{i}.attn.{qkv_conv_bn,proj_conv_bn}.{0,1}.*``, ``blocks.{i}.mlp.{fc1,fc2}.{0,1}.*``,
``head.{weight,bias}``.
Parity: ``spikingjelly/activation_based/model/spikformer.py:19-857``.

Two execution paths share the parameters: the module-by-module path (any device, any
backend) and, for CUDA tensors with the native backend, the fused channels-last path in
:mod:`spikingjelly_b200.models._spikformer_fused`.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..activation_based import base, functional, layer, neuron
from ..activation_based.layer.attention import SpikingSelfAttention

__all__ = ["Spikformer", "SpikformerBlock", "SpikformerConv2dBN", "SpikformerConv2dBNLIF", "SpikformerMLP",
           "SpikformerPatchStem", "spikformer_s", "spikformer_ti", "spikformer_8_512"]


class SpikformerConv2dBN(nn.Module):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, pool=False):
        super().__init__()
        mods = [nn.Conv2d(in_channels, out_channels, kernel_size, stride=stride, padding=padding, bias=False),
                nn.BatchNorm2d(out_channels)]
        if pool:
            mods.append(nn.MaxPool2d(kernel_size=3, stride=2, padding=1))
        self.block = layer.SeqToANNContainer(*mods)

    def forward(self, x_seq):
        return self.block(x_seq)

    def __spatial_split__(self):
        return tuple(self.block.children())


class SpikformerConv2dBNLIF(nn.Module, base.MultiStepModule):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, pool=False, backend="torch",
                 tau=2.0, detach_reset=True):
        super().__init__()
        self._step_mode = "m"
        self.conv_bn = SpikformerConv2dBN(in_channels, out_channels, kernel_size, stride, padding, pool)
        self.neuron = neuron.LIFNode(tau=tau, detach_reset=detach_reset, step_mode="m", backend=backend)

    def forward(self, x_seq):
        return self.neuron(self.conv_bn(x_seq))

    def __spatial_split__(self):
        return self.conv_bn, self.neuron


class SpikformerPatchStem(nn.Module, base.MultiStepModule):
    def __init__(self, img_size_h=224, img_size_w=224, patch_size=16, in_channels=3, embed_dims=256,
                 backend="torch", tau=2.0, detach_reset=True):
        super().__init__()
        if patch_size != 16:
            raise ValueError("The current SpikformerPatchStem uses a fixed 4-stage /16 patch pipeline; "
                             f"expected patch_size=16, but got {patch_size}.")
        self._step_mode = "m"
        self.image_size = (img_size_h, img_size_w)
        self.patch_size, self.embed_dims = patch_size, embed_dims
        dims = [embed_dims // 8, embed_dims // 4, embed_dims // 2, embed_dims]
        stages, c_in = [], in_channels
        for c_out in dims:
            stages.append(SpikformerConv2dBNLIF(c_in, c_out, 3, 1, 1, pool=True, backend=backend, tau=tau,
                                                detach_reset=detach_reset))
            c_in = c_out
        self.stages = nn.Sequential(*stages)
        self.positional_encoding = SpikformerConv2dBNLIF(embed_dims, embed_dims, 3, 1, 1, pool=False,
                                                         backend=backend, tau=tau, detach_reset=detach_reset)
        self.grid_size = (img_size_h // patch_size, img_size_w // patch_size)
        self.num_patches = self.grid_size[0] * self.grid_size[1]

    def forward(self, x_seq):
        x_seq = self.stages(x_seq)
        return self.positional_encoding(x_seq) + x_seq


class SpikformerMLP(nn.Module, base.MultiStepModule):
    def __init__(self, in_features, hidden_features, out_features, backend="torch", tau=2.0, detach_reset=True):
        super().__init__()
        self._step_mode = "m"
        self.fc1 = layer.SeqToANNContainer(nn.Conv1d(in_features, hidden_features, kernel_size=1, bias=False),
                                           nn.BatchNorm1d(hidden_features))
        self.neuron1 = neuron.LIFNode(tau=tau, detach_reset=detach_reset, step_mode="m", backend=backend)
        self.fc2 = layer.SeqToANNContainer(nn.Conv1d(hidden_features, out_features, kernel_size=1, bias=False),
                                           nn.BatchNorm1d(out_features))
        self.neuron2 = neuron.LIFNode(tau=tau, detach_reset=detach_reset, step_mode="m", backend=backend)

    def forward(self, x_seq):
        return self.neuron2(self.fc2(self.neuron1(self.fc1(x_seq))))

    def __spatial_split__(self):
        return self.fc1, self.neuron1, self.fc2, self.neuron2


class SpikformerBlock(nn.Module, base.MultiStepModule):
    def __init__(self, dim, num_heads, mlp_ratio=4.0, backend="torch", tau=2.0, detach_reset=True):
        super().__init__()
        self._step_mode = "m"
        self.attn = SpikingSelfAttention(dim=dim, num_heads=num_heads, backend=backend)
        self.mlp = SpikformerMLP(dim, int(dim * mlp_ratio), dim, backend=backend, tau=tau,
                                 detach_reset=detach_reset)

    def forward(self, x_seq):
        if x_seq.ndim != 5:
            raise ValueError(f"expected 5D input with shape [T, N, C, H, W], but got {x_seq.shape}")
        T, N, C, H, W = x_seq.shape
        tok = x_seq.flatten(3)
        tok = tok + self.attn(tok)
        tok = tok + self.mlp(tok)
        return tok.reshape(T, N, C, H, W).contiguous()


class Spikformer(nn.Module, base.MultiStepModule):
    def __init__(self, T=4, in_channels=3, img_size_h=224, img_size_w=224, patch_size=16, num_classes=1000,
                 embed_dims=256, num_heads=8, mlp_ratio=4.0, depths=4, backend="torch", tau=2.0,
                 detach_reset=True):
        super().__init__()
        self._step_mode = "m"
        self.T, self.num_classes, self.embed_dims = T, num_classes, embed_dims
        self.num_heads, self.depths = num_heads, depths
        self.patch_embed = SpikformerPatchStem(img_size_h, img_size_w, patch_size, in_channels, embed_dims,
                                               backend, tau, detach_reset)
        self.blocks = nn.ModuleList(SpikformerBlock(embed_dims, num_heads, mlp_ratio, backend, tau, detach_reset)
                                    for _ in range(depths))
        self.head = layer.Linear(embed_dims, num_classes, step_mode="m")
        self._init_weights()
        functional.set_step_mode(self, "m")
        #: use the fused channels-last CUDA path when input and backend allow it
        self.fused = True

    def _init_weights(self):
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Conv1d, nn.Conv2d)):
                nn.init.trunc_normal_(m.weight, std=0.02)
                if getattr(m, "bias", None) is not None:
                    nn.init.constant_(m.bias, 0.0)
            elif isinstance(m, (nn.BatchNorm1d, nn.BatchNorm2d)):
                nn.init.constant_(m.weight, 1.0)
                nn.init.constant_(m.bias, 0.0)

    def _to_sequence(self, x):
        if x.ndim == 4:
            return x.unsqueeze(0).repeat(self.T, 1, 1, 1, 1)
        if x.ndim == 5:
            return x
        raise ValueError("expected 4D image input [N, C, H, W] or 5D sequence input [T, N, C, H, W], "
                         f"but got {x.shape}")

    def forward_features(self, x_seq):
        x_seq = self.patch_embed(x_seq)
        for blk in self.blocks:
            x_seq = blk(x_seq)
        return x_seq.flatten(3).mean(dim=-1)

    def forward(self, x):
        if self.fused and x.is_cuda:
            from . import _spikformer_fused
            if _spikformer_fused.eligible(self, x):
                return _spikformer_fused.forward(self, x)
        return self.head(self.forward_features(self._to_sequence(x)))


def spikformer_ti(T=4, in_channels=3, img_size_h=224, img_size_w=224, num_classes=1000, backend="torch"):
    return Spikformer(T, in_channels, img_size_h, img_size_w, 16, num_classes, 256, 8, 4.0, 4, backend)


def spikformer_s(T=4, in_channels=3, img_size_h=224, img_size_w=224, num_classes=1000, backend="torch"):
    return Spikformer(T, in_channels, img_size_h, img_size_w, 16, num_classes, 384, 12, 4.0, 6, backend)


def spikformer_8_512(T=4, in_channels=3, img_size_h=224, img_size_w=224, num_classes=1000, backend="torch"):
    """Spikformer-8-512: 8 encoder blocks, embedding 512, 8 heads, MLP ratio 4."""
    return Spikformer(T, in_channels, img_size_h, img_size_w, 16, num_classes, 512, 8, 4.0, 8, backend)
