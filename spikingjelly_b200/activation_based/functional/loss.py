"""Losses for spike trains (``functional/loss.py:12-331``)."""
import torch
import torch.nn.functional as F
from torch import Tensor

__all__ = ["kernel_dot_product", "spike_similar_loss", "temporal_efficient_training_cross_entropy"]


def kernel_dot_product(x: Tensor, y: Tensor, kernel="linear", *args):
    """Gram matrix ``K[i, j] = k(x_i, y_j)`` for ``linear``, ``polynomial`` (degree
    ``args[0]``), ``sigmoid`` (slope ``args[0]``) or ``gaussian`` (sigma ``args[0]``)."""
    if kernel == "linear":
        return x.mm(y.t())
    if kernel == "polynomial":
        return x.mm(y.t()).pow(args[0])
    if kernel == "sigmoid":
        return torch.sigmoid(args[0] * x.mm(y.t()))
    if kernel == "gaussian":
        sigma = args[0]
        if sigma <= 0:
            raise ValueError(f"sigma must be positive for the Gaussian kernel, but got {sigma}")
        d = x.square().sum(1).unsqueeze(1) + y.square().sum(1).unsqueeze(0) - 2 * x.mm(y.t())
        return torch.exp(-d / (2 * sigma * sigma))
    raise NotImplementedError(kernel)


def spike_similar_loss(spikes: Tensor, labels: Tensor, kernel_type="linear", loss_type="mse", *args):
    """Make the similarity of output spike trains match label similarity:
    ``sim[i, j] = 1`` if samples ``i`` and ``j`` share a label."""
    spikes = spikes.flatten(start_dim=1)
    sim_p = kernel_dot_product(spikes, spikes, kernel_type, *args)
    if kernel_type == "linear":
        norm = spikes.norm(p=2, dim=1, keepdim=True)
        sim_p = sim_p / (norm.mm(norm.t()) + 1e-8)
    labels = labels.float()
    sim = labels.mm(labels.t()).clamp_max(1)
    if loss_type == "mse":
        return F.mse_loss(sim_p, sim)
    if loss_type == "l1":
        return F.l1_loss(sim_p, sim)
    if loss_type == "bce":
        return F.binary_cross_entropy(sim_p, sim)
    raise NotImplementedError(loss_type)


def temporal_efficient_training_cross_entropy(x_seq: Tensor, target: Tensor):
    """TET loss: cross entropy of every time step against the same target, averaged.
    ``x_seq`` is ``[T, N, C, *]``; ``target`` is ``[N, *]`` class indices."""
    logits = x_seq.permute(1, 2, 0, *range(3, x_seq.dim()))  # [N, C, T, *]
    T = logits.shape[2]
    reps = [1, T] + [1] * (logits.dim() - 3)
    return F.cross_entropy(logits, target.unsqueeze(1).repeat(reps))
