"""Legacy Tempotron kept for old checkpoints: the weight is ``fc.weight``, the loss a static method and
``"v_max"`` is squeezed (``spikingjelly/timing_based/orig_neuron.py:8-124``)."""
import torch
import torch.nn as nn

from .neuron import Tempotron as _Tempotron


class Tempotron(_Tempotron):
    def _make_layer(self, in_features, out_features):
        self.fc = nn.Linear(in_features, out_features, bias=False)

    def _summation(self):
        return self.fc

    @staticmethod
    def psp_kernel(t: torch.Tensor, tau, tau_s):
        return (torch.exp(-t / tau) - torch.exp(-t / tau_s)) * (t >= 0).float()

    @staticmethod
    def mse_loss(v_max, v_threshold, label, num_classes):
        wrong = ((v_max >= v_threshold).float() != nn.functional.one_hot(label, num_classes)).float()
        return torch.sum(torch.pow((v_max - v_threshold) * wrong, 2)) / label.shape[0]

    def forward(self, in_spikes: torch.Tensor, ret_type):
        out = super().forward(in_spikes, ret_type)
        return out.squeeze() if ret_type == "v_max" else out
