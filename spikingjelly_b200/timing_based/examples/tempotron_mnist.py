"""Tempotron on MNIST: every pixel is encoded by ``m`` Gaussian-tuned input neurons into one spike time in ``[0, T]``, a single
layer of ten tempotrons integrates the post-synaptic potentials and is trained on the maximum membrane potential (the neuron of
the right class should cross the threshold, the others should not).  Role of
``spikingjelly/timing_based/examples/tempotron_mnist.py``.

    python -m spikingjelly_b200.timing_based.examples.tempotron_mnist --synthetic --epochs 1
"""
import argparse

import torch
import torch.nn as nn
from torch.utils.data import DataLoader, TensorDataset

from .. import encoding, neuron


class Net(nn.Module):
    def __init__(self, m: int, T: int, pixels: int = 28 * 28):
        super().__init__()
        self.tempotron = neuron.Tempotron(pixels * m, 10, T)

    def forward(self, spike_times: torch.Tensor):
        """Maximum membrane potential of each output neuron while training, spikes (0 / 1) when evaluating."""
        return self.tempotron(spike_times, "v_max" if self.training else "spikes")


def blobs(n, seed):
    g = torch.Generator().manual_seed(99)
    prototypes = nn.functional.interpolate((torch.rand(10, 1, 4, 4, generator=g) > 0.5).float(), size=(28, 28), mode="nearest")
    g = torch.Generator().manual_seed(seed)
    labels = torch.randint(0, 10, (n,), generator=g)
    return TensorDataset((0.7 * prototypes[labels] + 0.3 * torch.rand(n, 1, 28, 28, generator=g)).clamp_(0, 1), labels)


def main(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    p.add_argument("--dataset-dir", default="./data/mnist")
    p.add_argument("--synthetic", action="store_true", help="generated digits instead of MNIST")
    p.add_argument("-b", "--batch-size", type=int, default=64)
    p.add_argument("-lr", "--learning-rate", type=float, default=1e-3)
    p.add_argument("-T", type=int, default=100, help="length of the encoding window")
    p.add_argument("-N", "--epochs", type=int, default=10)
    p.add_argument("-m", type=int, default=16, help="Gaussian-tuned input neurons per pixel")
    p.add_argument("--max-steps", type=int, default=None)
    args = p.parse_args(argv)
    device = torch.device(args.device)
    torch.manual_seed(0)
    if args.synthetic:
        train_set, test_set = blobs(1024, 1), blobs(256, 2)
    else:
        import torchvision
        tf = torchvision.transforms.ToTensor()
        train_set = torchvision.datasets.MNIST(args.dataset_dir, train=True, transform=tf, download=True)
        test_set = torchvision.datasets.MNIST(args.dataset_dir, train=False, transform=tf, download=True)
    train_loader = DataLoader(train_set, args.batch_size, shuffle=True, drop_last=True)
    test_loader = DataLoader(test_set, args.batch_size, shuffle=False)
    encoder = encoding.GaussianTuning(n=1, m=args.m, x_min=torch.zeros(1, device=device), x_max=torch.ones(1, device=device))
    net = Net(args.m, args.T).to(device)
    optimizer = torch.optim.SGD(net.parameters(), lr=args.learning_rate) if not args.synthetic else torch.optim.Adam(net.parameters(), lr=args.learning_rate)

    def encode(img):                                   # [B, 1, 28, 28] -> spike times [B, 784 * m]
        return encoder.encode(img.to(device).view(img.shape[0], 1, -1), args.T).view(img.shape[0], -1)
    history, step = [], 0
    for epoch in range(args.epochs):
        net.train()
        for img, label in train_loader:
            v_max = net(encode(img))
            loss = net.tempotron.mse_loss(v_max, label.to(device))
            optimizer.zero_grad(set_to_none=True)
            loss.backward()
            optimizer.step()
            step += 1
            if args.max_steps is not None and step >= args.max_steps:
                break
        net.eval()
        hit = total = 0
        with torch.no_grad():
            for img, label in test_loader:
                net.train()                            # the read-out uses the potentials: the largest maximum wins
                v_max = net(encode(img))
                net.eval()
                hit += int((v_max.argmax(1).cpu() == label).sum())
                total += label.numel()
        history.append({"epoch": epoch, "loss": float(loss), "test_accuracy": hit / total})
        print(history[-1], flush=True)
        if args.max_steps is not None and step >= args.max_steps:
            break
    return history


if __name__ == "__main__":
    main()
