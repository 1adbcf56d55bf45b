"""Gaussian receptive-field (population) encoding of real values into spike times
(``spikingjelly/timing_based/encoding.py:6-132``)."""
import torch

__all__ = ["GaussianTuning"]


class GaussianTuning:
    """``n`` input features, each seen by ``m`` Gaussian tuning curves whose centres tile ``[x_min, x_max]``
    (``mu_i = x_min + (2i - 3) / 2 * range / (m - 2)``, ``sigma = range / (1.5 (m - 2))``).  A strong response
    fires early: ``t = round(max_spike_time * (1 - response))``; responses too weak to fire by
    ``max_spike_time`` are encoded as ``-1``."""

    def __init__(self, n: int, m: int, x_min: torch.Tensor, x_max: torch.Tensor) -> None:
        if n <= 0:
            raise ValueError("n must be a positive integer.")
        if m <= 2:
            raise ValueError("m must be greater than 2.")
        if x_min.shape != (n,) or x_max.shape != (n,):
            raise ValueError(f"x_min and x_max must both have shape ({n},), but got {x_min.shape} and {x_max.shape}.")
        if not torch.all(x_min < x_max):
            raise ValueError("All elements of x_min must be less than x_max.")
        self.n, self.m = n, m
        i = torch.arange(1, m + 1, device=x_min.device, dtype=torch.float32).unsqueeze(0)
        span = (x_max - x_min).unsqueeze(-1)
        self.mu = x_min.unsqueeze(-1) + (2 * i - 3) * span / (2 * (m - 2))
        self.sigma2 = (span / (1.5 * (m - 2))).square().repeat(1, m)

    def encode(self, x: torch.Tensor, max_spike_time: int = 50) -> torch.Tensor:
        """``[batch, n, k]`` -> spike times ``[batch, n, k, m]``."""
        if x.dim() != 3 or x.shape[1] != self.n:
            raise AssertionError(f"x must have shape [batch_size, {self.n}, samples_count], but got {tuple(x.shape)}.")
        max_spike_time = max_spike_time or 100
        response = torch.exp(-(x.unsqueeze(-1) - self.mu[None, :, None, :]).square() / (2 * self.sigma2[None, :, None, :]))
        times = (max_spike_time * (1 - response)).round()
        return times.masked_fill(times >= max_spike_time, -1)
