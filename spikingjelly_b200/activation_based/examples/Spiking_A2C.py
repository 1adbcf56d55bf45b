"""Advantage actor-critic and PPO (clipped surrogate) on cart-pole with a spiking actor-critic network (the reference's
``examples/Spiking_A2C.py`` and ``examples/Spiking_PPO.py``) or an ordinary MLP (``examples/A2C.py``, ``examples/PPO.py``).

Spiking network: Linear -> IF -> two heads (Linear -> non-spiking LIF read-out, maximum potential over ``T`` steps): action
logits and state value.  A2C updates after every episode from the Monte-Carlo returns; PPO collects ``--horizon`` steps, then
runs ``--ppo-epochs`` passes of clipped-ratio updates over mini-batches with generalised advantage estimation.

    python -m spikingjelly_b200.activation_based.examples.Spiking_A2C --episodes 300 [--ppo] [--ann] [--builtin-env]
"""
from __future__ import annotations

import argparse
import random

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import functional, layer, neuron
from . import _cartpole as env_lib


class SpikingActorCritic(nn.Module):
    def __init__(self, n_states: int, hidden: int, n_actions: int, T: int = 16):
        super().__init__()
        self.T = T
        self.body = nn.Sequential(layer.Linear(n_states, hidden, step_mode="m"), neuron.IFNode(step_mode="m"))
        self.actor = nn.Sequential(layer.Linear(hidden, n_actions, step_mode="m"), neuron.NonSpikingLIFNode(tau=2.0, decode="max-mem"))
        self.critic = nn.Sequential(layer.Linear(hidden, 1, step_mode="m"), neuron.NonSpikingLIFNode(tau=2.0, decode="max-mem"))

    def forward(self, x):
        s = self.body(x.unsqueeze(0).expand(self.T, -1, -1))
        logits, value = self.actor(s), self.critic(s)
        functional.reset_net(self)
        return logits, value.squeeze(-1)


class ActorCritic(nn.Module):
    def __init__(self, n_states: int, hidden: int, n_actions: int):
        super().__init__()
        self.body = nn.Sequential(nn.Linear(n_states, hidden), nn.ReLU())
        self.actor, self.critic = nn.Linear(hidden, n_actions), nn.Linear(hidden, 1)

    def forward(self, x):
        h = self.body(x)
        return self.actor(h), self.critic(h).squeeze(-1)


def _returns(rewards, dones, gamma, last_value=0.0):
    out, run = [], last_value
    for r, d in zip(reversed(rewards), reversed(dones)):
        run = r + gamma * run * (0.0 if d else 1.0)
        out.append(run)
    return list(reversed(out))


def _gae(rewards, values, dones, last_value, gamma, lam):
    adv, run = [], 0.0
    values = values + [last_value]
    for t in reversed(range(len(rewards))):
        alive = 0.0 if dones[t] else 1.0
        delta = rewards[t] + gamma * values[t + 1] * alive - values[t]
        run = delta + gamma * lam * alive * run
        adv.append(run)
    adv.reverse()
    return adv, [a + v for a, v in zip(adv, values[:-1])]


def main(argv=None) -> dict:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--episodes", type=int, default=300)
    p.add_argument("--hidden", type=int, default=128)
    p.add_argument("-T", type=int, default=16)
    p.add_argument("--ann", action="store_true")
    p.add_argument("--ppo", action="store_true", help="PPO with clipped ratio and GAE instead of per-episode A2C")
    p.add_argument("--horizon", type=int, default=256)
    p.add_argument("--ppo-epochs", type=int, default=4)
    p.add_argument("--minibatch", type=int, default=64)
    p.add_argument("--clip", type=float, default=0.2)
    p.add_argument("--lam", type=float, default=0.95)
    p.add_argument("--gamma", type=float, default=0.99)
    p.add_argument("--entropy", type=float, default=0.01)
    p.add_argument("--lr", type=float, default=3e-3)
    p.add_argument("--builtin-env", action="store_true")
    p.add_argument("--device", default="cpu")
    p.add_argument("--seed", type=int, default=1)
    a = p.parse_args(argv)
    random.seed(a.seed)
    torch.manual_seed(a.seed)
    device = torch.device(a.device)
    env = env_lib.make_env(a.seed, a.builtin_env)
    net = (ActorCritic(4, a.hidden, 2) if a.ann else SpikingActorCritic(4, a.hidden, 2, a.T)).to(device)
    opt = torch.optim.Adam(net.parameters(), lr=a.lr)
    durations, best = [], 0
    buf = {k: [] for k in ("s", "a", "logp", "v", "r", "d")}

    def act(state):
        with torch.no_grad():
            logits, value = net(state)
        dist = torch.distributions.Categorical(logits=logits)
        action = dist.sample()
        return int(action), float(dist.log_prob(action)), float(value)

    def a2c_update():
        states, actions = torch.cat(buf["s"]), torch.tensor(buf["a"], device=device)
        ret = torch.tensor(_returns(buf["r"], buf["d"], a.gamma), device=device)
        logits, values = net(states)
        dist = torch.distributions.Categorical(logits=logits)
        adv = ret - values.detach()
        loss = -(dist.log_prob(actions) * adv).mean() + 0.5 * F.mse_loss(values, ret) - a.entropy * dist.entropy().mean()
        opt.zero_grad(); loss.backward(); nn.utils.clip_grad_norm_(net.parameters(), 1.0); opt.step()

    def ppo_update(last_value):
        adv, ret = _gae(buf["r"], buf["v"], buf["d"], last_value, a.gamma, a.lam)
        states, actions = torch.cat(buf["s"]), torch.tensor(buf["a"], device=device)
        old_logp, adv, ret = torch.tensor(buf["logp"], device=device), torch.tensor(adv, device=device), torch.tensor(ret, device=device)
        adv = (adv - adv.mean()) / (adv.std() + 1e-8)
        n = states.shape[0]
        for _ in range(a.ppo_epochs):
            perm = torch.randperm(n, device=device)
            for i in range(0, n, a.minibatch):
                idx = perm[i:i + a.minibatch]
                logits, values = net(states[idx])
                dist = torch.distributions.Categorical(logits=logits)
                ratio = (dist.log_prob(actions[idx]) - old_logp[idx]).exp()
                surr = torch.min(ratio * adv[idx], ratio.clamp(1 - a.clip, 1 + a.clip) * adv[idx])
                loss = -surr.mean() + 0.5 * F.mse_loss(values, ret[idx]) - a.entropy * dist.entropy().mean()
                opt.zero_grad(); loss.backward(); nn.utils.clip_grad_norm_(net.parameters(), 0.5); opt.step()

    for ep in range(a.episodes):
        state = torch.tensor([env_lib.reset_env(env)], dtype=torch.float32, device=device)
        t = 0
        while True:
            action, logp, value = act(state)
            obs, reward, over, fell = env_lib.step_env(env, action)
            t += 1
            for k, v in zip(("s", "a", "logp", "v", "r", "d"), (state, action, logp, value, reward, fell or over)):
                buf[k].append(v)
            state = torch.tensor([obs], dtype=torch.float32, device=device)
            if a.ppo and len(buf["r"]) >= a.horizon:
                ppo_update(0.0 if (fell or over) else act(state)[2])
                buf = {k: [] for k in buf}
            if over:
                break
        if not a.ppo:
            a2c_update()
            buf = {k: [] for k in buf}
        durations.append(t)
        best = max(best, t)
        if ep % 20 == 0 or ep + 1 == a.episodes:
            print(f"episode {ep}: {t} steps (best {best}, mean of last 10 {sum(durations[-10:]) / len(durations[-10:]):.1f})")
    return {"episodes": a.episodes, "best": best, "last_mean": sum(durations[-10:]) / len(durations[-10:])}


if __name__ == "__main__":
    main()
