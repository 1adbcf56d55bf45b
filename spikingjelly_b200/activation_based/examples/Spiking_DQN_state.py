"""Deep Q-learning on cart-pole states with a spiking Q-network (the reference's ``examples/Spiking_DQN_state.py``) or an
ordinary MLP (``examples/DQN_state.py``): replay memory, epsilon-greedy policy, target network, Huber loss.

The spiking network is Linear -> IF -> Linear -> non-spiking LIF read-out: the state is presented for ``T`` steps and the
Q-values are the maximum membrane potential of the read-out neurons over those steps.

    python -m spikingjelly_b200.activation_based.examples.Spiking_DQN_state --episodes 200 [--ann] [--builtin-env]
"""
from __future__ import annotations

import argparse
import math
import random
from collections import deque, namedtuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import functional, layer, neuron
from . import _cartpole as env_lib

Transition = namedtuple("Transition", ("state", "action", "next_state", "reward"))


class ReplayMemory:
    def __init__(self, capacity: int, seed: int = 0):
        self.buf = deque(maxlen=capacity)
        self.rng = random.Random(seed)

    def push(self, *args):
        self.buf.append(Transition(*args))

    def sample(self, n: int):
        return self.rng.sample(self.buf, n)

    def __len__(self):
        return len(self.buf)


class NonSpikingLIFMax(neuron.NonSpikingLIFNode):
    """Read-out: integrates without firing; the forward value is the largest potential seen over the sequence."""

    def __init__(self, tau: float = 2.0):
        super().__init__(tau=tau, decode="max-mem")


class DQSN(nn.Module):
    def __init__(self, n_states: int, hidden: int, n_actions: int, T: int = 16):
        super().__init__()
        self.T = T
        self.fc = nn.Sequential(layer.Linear(n_states, hidden, step_mode="m"), neuron.IFNode(step_mode="m"),
                                layer.Linear(hidden, n_actions, step_mode="m"), NonSpikingLIFMax(2.0))

    def forward(self, x):                                        # [N, states] -> Q [N, actions]
        q = self.fc(x.unsqueeze(0).expand(self.T, -1, -1))
        functional.reset_net(self)
        return q


class DQN(nn.Module):
    def __init__(self, n_states: int, hidden: int, n_actions: int):
        super().__init__()
        self.fc = nn.Sequential(nn.Linear(n_states, hidden), nn.ReLU(), nn.Linear(hidden, n_actions))

    def forward(self, x):
        return self.fc(x)


def main(argv=None) -> dict:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--episodes", type=int, default=200)
    p.add_argument("--hidden", type=int, default=256)
    p.add_argument("-T", type=int, default=16)
    p.add_argument("--ann", action="store_true", help="ordinary MLP Q-network instead of the spiking one")
    p.add_argument("--builtin-env", action="store_true", help="use the built-in cart-pole even if gym is installed")
    p.add_argument("--batch-size", type=int, default=128)
    p.add_argument("--gamma", type=float, default=0.999)
    p.add_argument("--eps-start", type=float, default=0.9)
    p.add_argument("--eps-end", type=float, default=0.05)
    p.add_argument("--eps-decay", type=float, default=200.0)
    p.add_argument("--target-update", type=int, default=10)
    p.add_argument("--lr", type=float, default=1e-3)
    p.add_argument("--device", default="cpu")
    p.add_argument("--seed", type=int, default=1)
    a = p.parse_args(argv)
    random.seed(a.seed)
    torch.manual_seed(a.seed)
    device = torch.device(a.device)
    env = env_lib.make_env(a.seed, a.builtin_env)
    make = (lambda: DQN(4, a.hidden, 2)) if a.ann else (lambda: DQSN(4, a.hidden, 2, a.T))
    policy, target = make().to(device), make().to(device)
    target.load_state_dict(policy.state_dict())
    target.eval()
    opt = torch.optim.Adam(policy.parameters(), lr=a.lr)
    memory = ReplayMemory(10000, a.seed)
    steps_done, durations, best = 0, [], 0

    def select_action(state):
        nonlocal steps_done
        eps = a.eps_end + (a.eps_start - a.eps_end) * math.exp(-steps_done / a.eps_decay)
        steps_done += 1
        if random.random() > eps:
            with torch.no_grad():
                return int(policy(state).argmax(1))
        return random.randrange(2)

    def optimize():
        if len(memory) < a.batch_size:
            return None
        batch = Transition(*zip(*memory.sample(a.batch_size)))
        alive = torch.tensor([s is not None for s in batch.next_state], device=device)
        nxt = torch.cat([s for s in batch.next_state if s is not None]) if alive.any() else None
        state, action, reward = torch.cat(batch.state), torch.tensor(batch.action, device=device).unsqueeze(1), torch.tensor(batch.reward, device=device)
        q = policy(state).gather(1, action).squeeze(1)
        v_next = torch.zeros(a.batch_size, device=device)
        if nxt is not None:
            with torch.no_grad():
                v_next[alive] = target(nxt).max(1).values
        loss = F.smooth_l1_loss(q, reward + a.gamma * v_next)
        opt.zero_grad()
        loss.backward()
        for prm in policy.parameters():
            if prm.grad is not None:
                prm.grad.clamp_(-1, 1)
        opt.step()
        return float(loss)

    for ep in range(a.episodes):
        state = torch.tensor([env_lib.reset_env(env)], dtype=torch.float32, device=device)
        t = 0
        while True:
            action = select_action(state)
            obs, _, over, fell = env_lib.step_env(env, action)
            t += 1
            # shaped reward of the reference script: distance from the track's edge and from the angle limit
            x, _, th, _ = obs
            reward = (2.4 - abs(x)) / 2.4 - 0.8 + (0.2095 - abs(th)) / 0.2095 - 0.5
            nxt = None if fell else torch.tensor([obs], dtype=torch.float32, device=device)
            memory.push(state, action, nxt, float(reward))
            state = nxt if nxt is not None else state
            optimize()
            if over:
                break
        durations.append(t)
        best = max(best, t)
        if ep % a.target_update == 0:
            target.load_state_dict(policy.state_dict())
        if ep % 10 == 0 or ep + 1 == a.episodes:
            print(f"episode {ep}: {t} steps (best {best}, mean of last 10 {sum(durations[-10:]) / len(durations[-10:]):.1f})")
    return {"episodes": a.episodes, "best": best, "last_mean": sum(durations[-10:]) / len(durations[-10:])}


if __name__ == "__main__":
    main()
