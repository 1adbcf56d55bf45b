"""Small ReLU CNN for MNIST used by the conversion examples (conv-BN-ReLU-pool x3, linear head).
Parity: ``spikingjelly/activation_based/ann2snn/sample_models/mnist_cnn.py:1-45``."""
import torch.nn as nn

__all__ = ["CNN"]


class CNN(nn.Module):
    def __init__(self):
        super().__init__()
        def stage(cin, cout, pool):
            return [nn.Conv2d(cin, cout, 3, 1), nn.BatchNorm2d(cout, eps=1e-3), nn.ReLU(), nn.AvgPool2d(pool, pool)]
        self.network = nn.Sequential(*stage(1, 32, 2), *stage(32, 32, 2), *stage(32, 32, 2), nn.Flatten(), nn.Linear(32, 10), nn.ReLU())

    def forward(self, x):
        return self.network(x)
