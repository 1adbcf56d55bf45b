"""Deep spiking Q-network on image observations (Chen et al., "Deep Reinforcement Learning with Spiking Q-learning", 2022):
Conv - LIF - Conv - LIF - Linear - LIF - Linear - non-spiking LIF, the frame stack presented for ``T`` steps and the
Q-values read as the maximum membrane potential of the non-spiking output neurons.  Counterpart of the reference's
``examples/DSQN/train.py`` (there on Atari through ``ptan``); here the agent plays a dependency-free pixel game, *catch* (a
ball falls down a ``size x size`` screen, a three-pixel paddle moves left / stays / moves right, reward +1 / -1 when the ball
reaches the bottom row), so the script runs without the Arcade Learning Environment.  Double-DQN targets, Huber loss, a
target network synchronised every ``--sync`` steps, linear epsilon decay.

    python -m spikingjelly_b200.activation_based.examples.DSQN --frames 20000 -T 8
"""
from __future__ import annotations

import argparse
import random
from collections import deque

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import functional, layer, neuron, surrogate

__all__ = ["Catch", "DSQN", "train"]


class Catch:
    n_actions = 3

    def __init__(self, size: int = 12, seed: int = 0):
        self.size, self.rng = size, random.Random(seed)
        self.reset()

    def _frame(self) -> np.ndarray:
        f = np.zeros((1, self.size, self.size), np.float32)
        f[0, self.ball_y, self.ball_x] = 1.0
        f[0, self.size - 1, max(self.paddle - 1, 0):self.paddle + 2] = 1.0
        return f

    def reset(self) -> np.ndarray:
        self.ball_x, self.ball_y, self.paddle = self.rng.randrange(self.size), 0, self.size // 2
        return self._frame()

    def step(self, action: int):
        self.paddle = min(max(self.paddle + (action - 1), 1), self.size - 2)
        self.ball_y += 1
        done = self.ball_y == self.size - 1
        reward = (1.0 if abs(self.ball_x - self.paddle) <= 1 else -1.0) if done else 0.0
        return self._frame(), reward, done


class DSQN(nn.Module):
    """``forward(frames [B, C, H, W]) -> Q [B, actions]``: the same frames are fed for ``T`` steps."""

    def __init__(self, in_channels: int, size: int, n_actions: int, T: int = 8, hidden: int = 128, backend: str = "torch"):
        super().__init__()
        self.T = T
        sg = surrogate.ATan()
        lif = lambda: neuron.LIFNode(tau=2.0, surrogate_function=sg, detach_reset=True, backend=backend)
        self.features = nn.Sequential(layer.Conv2d(in_channels, 16, 3, padding=1), lif(), layer.Conv2d(16, 32, 3, stride=2, padding=1), lif(),
                                      layer.Flatten())
        side = (size + 1) // 2
        self.head = nn.Sequential(layer.Linear(32 * side * side, hidden), lif(), layer.Linear(hidden, n_actions))
        self.readout = neuron.NonSpikingLIFNode(tau=2.0, decode="max-mem")
        functional.set_step_mode(self, "m")

    def forward(self, frames: torch.Tensor) -> torch.Tensor:
        seq = frames.unsqueeze(0).expand(self.T, *frames.shape)
        q = self.readout(self.head(self.features(seq)))
        functional.reset_net(self)
        return q


def train(frames: int = 20000, T: int = 8, size: int = 12, batch_size: int = 32, gamma: float = 0.95, lr: float = 1e-3, sync: int = 500,
          buffer: int = 10000, start: int = 500, eps_final: float = 0.05, eps_frames: int = 10000, seed: int = 0, device: str = "cpu",
          log_every: int = 2000, quiet: bool = False):
    """Returns ``(network, list of episode rewards)``."""
    torch.manual_seed(seed)
    rng = random.Random(seed)
    dev = torch.device(device)
    env = Catch(size, seed)
    net = DSQN(1, size, env.n_actions, T, backend="cuda" if dev.type == "cuda" else "torch").to(dev)
    target = DSQN(1, size, env.n_actions, T, backend="cuda" if dev.type == "cuda" else "torch").to(dev)
    target.load_state_dict(net.state_dict())
    opt = torch.optim.Adam(net.parameters(), lr=lr)
    memory: deque = deque(maxlen=buffer)
    obs, rewards = env.reset(), []
    for frame in range(frames):
        eps = max(eps_final, 1.0 - frame / eps_frames * (1.0 - eps_final))
        if rng.random() < eps:
            action = rng.randrange(env.n_actions)
        else:
            with torch.no_grad():
                action = int(net(torch.as_tensor(obs, device=dev).unsqueeze(0)).argmax(1))
        nxt, reward, done = env.step(action)
        memory.append((obs, action, reward, nxt, done))
        obs = env.reset() if done else nxt
        if done:
            rewards.append(reward)
        if len(memory) >= max(start, batch_size):
            batch = rng.sample(memory, batch_size)
            o, a, r, o2, d = (np.stack(x) if isinstance(x[0], np.ndarray) else np.asarray(x) for x in zip(*batch))
            o, o2 = torch.as_tensor(o, device=dev), torch.as_tensor(o2, device=dev)
            a, r, d = torch.as_tensor(a, device=dev), torch.as_tensor(r, device=dev, dtype=torch.float32), torch.as_tensor(d, device=dev)
            with torch.no_grad():                                   # double DQN: the online net picks, the target net evaluates
                best = net(o2).argmax(1, keepdim=True)
                nxt_q = target(o2).gather(1, best).squeeze(1)
                want = r + gamma * nxt_q * (~d)
            loss = F.smooth_l1_loss(net(o).gather(1, a.view(-1, 1)).squeeze(1), want)
            opt.zero_grad(set_to_none=True)
            loss.backward()
            opt.step()
        if (frame + 1) % sync == 0:
            target.load_state_dict(net.state_dict())
        if not quiet and (frame + 1) % log_every == 0 and rewards:
            print(f"frame {frame + 1}: episodes {len(rewards)}, catch rate of the last 50 = {np.mean([x > 0 for x in rewards[-50:]]):.2f}")
    return net, rewards


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--frames", type=int, default=20000)
    ap.add_argument("-T", type=int, default=8)
    ap.add_argument("--size", type=int, default=12)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    return train(a.frames, a.T, a.size, device=a.device, seed=a.seed)


if __name__ == "__main__":
    main()
