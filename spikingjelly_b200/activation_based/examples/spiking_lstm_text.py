"""Character-level sequence classification with ``rnn.SpikingLSTM`` (the reference's ``examples/spiking_lstm_text.py`` classifies
surnames by language): a word is a sequence of one-hot characters, the spiking LSTM reads it one character per time step and a
linear layer maps the last hidden state to the class.

Without the names data set (``--data-dir`` with one ``<Language>.txt`` file of names per class, as in the PyTorch tutorial the
reference follows) the script generates words from class-specific character distributions (``--synthetic``).

    python -m spikingjelly_b200.activation_based.examples.spiking_lstm_text --synthetic --steps 300
"""
from __future__ import annotations

import argparse
import glob
import os
import random
import string
import unicodedata

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import functional, rnn

LETTERS = string.ascii_letters + " .,;'"


def to_ascii(s: str) -> str:
    return "".join(c for c in unicodedata.normalize("NFD", s) if unicodedata.category(c) != "Mn" and c in LETTERS)


def word_to_tensor(word: str) -> torch.Tensor:
    """``[len(word), 1, n_letters]`` one-hot."""
    idx = torch.tensor([LETTERS.find(c) for c in word])
    return F.one_hot(idx, len(LETTERS)).float().unsqueeze(1)


def load_names(root: str):
    data = {}
    for path in sorted(glob.glob(os.path.join(root, "*.txt"))):
        with open(path, encoding="utf-8") as f:
            names = [to_ascii(line.strip()) for line in f if line.strip()]
        data[os.path.splitext(os.path.basename(path))[0]] = [n for n in names if n]
    if not data:
        raise FileNotFoundError(f"no <Language>.txt files under {root}")
    return data


def synthetic_names(classes: int = 4, per_class: int = 200, seed: int = 0):
    rng = random.Random(seed)
    letters = string.ascii_lowercase
    data = {}
    for c in range(classes):
        favoured = letters[c * 5:(c + 1) * 5]                       # each "language" over-uses five letters
        words = []
        for _ in range(per_class):
            n = rng.randint(4, 9)
            words.append("".join(rng.choice(favoured) if rng.random() < 0.7 else rng.choice(letters) for _ in range(n)))
        data[f"lang{c}"] = words
    return data


class Net(nn.Module):
    def __init__(self, n_input: int, n_hidden: int, n_output: int):
        super().__init__()
        self.lstm = rnn.SpikingLSTM(n_input, n_hidden, 1)
        self.fc = nn.Linear(n_hidden, n_output)

    def forward(self, x):                                            # [T, N, letters]
        y, _ = self.lstm(x)
        return self.fc(y[-1])


def main(argv=None) -> dict:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--data-dir", default="")
    p.add_argument("--synthetic", action="store_true")
    p.add_argument("--hidden", type=int, default=128)
    p.add_argument("--steps", type=int, default=1000)
    p.add_argument("--lr", type=float, default=5e-3)
    p.add_argument("--device", default="cpu")
    p.add_argument("--seed", type=int, default=0)
    a = p.parse_args(argv)
    random.seed(a.seed)
    torch.manual_seed(a.seed)
    device = torch.device(a.device)
    data = synthetic_names(seed=a.seed) if a.synthetic or not a.data_dir else load_names(a.data_dir)
    classes = sorted(data)
    split = {c: (ws[: int(0.8 * len(ws))], ws[int(0.8 * len(ws)):]) for c, ws in data.items()}
    net = Net(len(LETTERS), a.hidden, len(classes)).to(device)
    opt = torch.optim.Adam(net.parameters(), lr=a.lr)
    running, log = 0.0, []
    for step in range(1, a.steps + 1):
        ci = random.randrange(len(classes))
        word = random.choice(split[classes[ci]][0])
        out = net(word_to_tensor(word).to(device))
        loss = F.cross_entropy(out, torch.tensor([ci], device=device))
        opt.zero_grad()
        loss.backward()
        opt.step()
        functional.reset_net(net)
        running += loss.item()
        if step % max(a.steps // 5, 1) == 0:
            log.append(running / max(a.steps // 5, 1))
            print(f"step {step}: mean loss {log[-1]:.4f}")
            running = 0.0
    net.eval()
    correct = total = 0
    with torch.no_grad():
        for ci, c in enumerate(classes):
            for word in split[c][1][:50]:
                correct += int(net(word_to_tensor(word).to(device)).argmax(1).item() == ci)
                total += 1
                functional.reset_net(net)
    acc = correct / max(total, 1)
    print(f"test accuracy {acc:.3f} over {total} words, {len(classes)} classes")
    return {"first_loss": log[0] if log else float("nan"), "last_loss": log[-1] if log else float("nan"), "test_acc": acc}


if __name__ == "__main__":
    main()
