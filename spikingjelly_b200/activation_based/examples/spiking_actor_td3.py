"""Hybrid TD3 with a fully spiking actor: population-coded observations, a spiking MLP, and a population decoder whose last
layer has intralayer connections (ILC-SAN, Chen et al., TNNLS 2024) or learnable coloured noise in every layer (NoisySAN,
Chen et al., 2024).  The critics are ordinary MLPs.  Counterpart of the reference's ``examples/ILC-SAN/`` and
``examples/NoisySAN/`` (``ilcsan.py``, ``noisysan.py``, ``hybrid_td3_cuda_norm.py``, ``replay_buffer_norm.py``), written as
one script with two actor kinds and a dependency-free pendulum so that it runs without ``gym`` / MuJoCo:

    python -m spikingjelly_b200.activation_based.examples.spiking_actor_td3 --actor ilc --steps 4000
    python -m spikingjelly_b200.activation_based.examples.spiking_actor_td3 --actor noisy --env Pendulum-v1   # if gymnasium is present

Observation normalisation (running mean / variance kept by the replay buffer), target-policy smoothing, delayed policy
updates and Polyak averaging follow TD3; the actor runs ``--spike-ts`` time steps per decision and is reset after it.
"""
from __future__ import annotations

import argparse
import copy
import math
import random
from collections import OrderedDict
from typing import Tuple

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import encoding, functional, layer, neuron, surrogate

__all__ = ["Pendulum", "SpikingActor", "Critic", "ReplayBuffer", "HybridTD3", "train"]


class Pendulum:
    """Torque-limited pendulum swing-up (the classic control task): observation ``(cos th, sin th, th_dot)``, one action in
    ``[-2, 2]``, reward ``-(th^2 + 0.1 th_dot^2 + 0.001 a^2)``, 200 steps per episode."""
    obs_dim, act_dim, act_limit, max_steps = 3, 1, 2.0, 200

    def __init__(self, seed: int = 0):
        self.rng = random.Random(seed)
        self.th = self.th_dot = 0.0
        self.t = 0

    def _obs(self):
        return np.array([math.cos(self.th), math.sin(self.th), self.th_dot], dtype=np.float32)

    def reset(self):
        self.th, self.th_dot, self.t = self.rng.uniform(-math.pi, math.pi), self.rng.uniform(-1.0, 1.0), 0
        return self._obs()

    def step(self, action):
        a = float(np.clip(np.asarray(action).reshape(-1)[0], -self.act_limit, self.act_limit))
        th = ((self.th + math.pi) % (2 * math.pi)) - math.pi
        cost = th ** 2 + 0.1 * self.th_dot ** 2 + 0.001 * a ** 2
        self.th_dot = float(np.clip(self.th_dot + (3 * 10.0 / 2 * math.sin(self.th) + 3.0 * a) * 0.05, -8.0, 8.0))
        self.th += self.th_dot * 0.05
        self.t += 1
        return self._obs(), -cost, self.t >= self.max_steps


class SpikingActor(nn.Module):
    """Population encoder -> spiking MLP (current-based LIF neurons) -> decoding population -> action in
    ``[-act_limit, act_limit]``.  ``kind="ilc"``: the decoding population has intralayer connections and the action is read
    from its last membrane potentials through a grouped 1-D convolution; ``kind="noisy"``: every layer injects learnable
    coloured noise and a noisy non-spiking neuron integrates the decoded currents."""

    def __init__(self, obs_dim: int, act_dim: int, act_limit: float, kind: str = "ilc", hidden=(64, 64), enc_pop: int = 10, dec_pop: int = 10,
                 spike_ts: int = 5, mean_range=(-3.0, 3.0), std: float = math.sqrt(0.15)):
        super().__init__()
        if kind not in ("ilc", "noisy"):
            raise ValueError("kind must be 'ilc' or 'noisy'")
        self.kind, self.act_dim, self.dec_pop, self.spike_ts, self.act_limit = kind, act_dim, dec_pop, spike_ts, act_limit
        self.encoder = encoding.PopSpikeEncoderDeterministic(obs_dim, enc_pop, spike_ts, mean_range, std)
        sg = surrogate.Rect()
        mods, width = OrderedDict(), obs_dim * enc_pop
        for i, h in enumerate(hidden):
            mods[f"Linear{i}"] = layer.Linear(width, h)
            mods[f"Node{i}"] = neuron.CUBALIFNode(surrogate_function=sg) if kind == "ilc" else \
                neuron.NoisyCUBALIFNode(h, T=spike_ts, surrogate_function=sg)
            width = h
        mods["LinearOut"] = layer.Linear(width, act_dim * dec_pop)
        mods["NodeOut"] = neuron.ILCCUBALIFNode(act_dim, dec_pop, surrogate_function=sg) if kind == "ilc" else \
            neuron.NoisyILCCUBALIFNode(act_dim, dec_pop, T=spike_ts, surrogate_function=sg)
        self.body = nn.Sequential(mods)
        functional.set_step_mode(self.body, "m")
        self.group_readout = nn.Conv1d(act_dim, act_dim, dec_pop, groups=act_dim)
        if kind == "noisy":
            self.integrator = neuron.NoisyNonSpikingIFNode(act_dim, T=spike_ts)
            functional.set_step_mode(self.integrator, "m")

    # -- coloured noise of the noisy actor: sampled per episode, stored with every transition, replayed in the update ------
    def _noisy(self):
        return [m for m in self.modules() if hasattr(m, "reset_noise") and m is not self]

    def reset_noise(self, num_steps: int) -> None:
        for m in self._noisy():
            m.reset_noise(num_steps)

    def set_noise(self, enabled: bool) -> None:
        for m in self._noisy():
            m.is_training = enabled

    def noise_length(self) -> int:
        return sum(2 * m.num_node if hasattr(m, "eps_v_seq") or hasattr(m, "sigma_v") else m.num_node for m in self._noisy())

    def get_colored_noise(self) -> torch.Tensor:
        """``[T, noise_length]``: the noise the last forward used, every noisy module's share side by side."""
        parts = [m.get_colored_noise() for m in self._noisy()]
        return torch.cat(parts, dim=1) if parts else torch.zeros(self.spike_ts, 0)

    def load_colored_noise(self, cn: torch.Tensor) -> None:
        """``cn``: ``[B, T, noise_length]`` as stored by :meth:`get_colored_noise` per transition."""
        at = 0
        for m in self._noisy():
            n = 2 * m.num_node if hasattr(m, "sigma_v") else m.num_node
            m.load_colored_noise(cn[:, :, at:at + n])
            at += n

    def cancel_load(self) -> None:
        for m in self._noisy():
            m.cancel_load()

    def forward(self, obs: torch.Tensor) -> torch.Tensor:
        spikes = self.body(self.encoder(obs))                                     # [T, B, act_dim * dec_pop]
        if self.kind == "ilc":
            v = self.body.NodeOut.v                                               # last membrane potentials of the decoding population
            raw = self.group_readout(v.view(-1, self.act_dim, self.dec_pop)).view(-1, self.act_dim)
        else:
            T, B = spikes.shape[:2]
            cur = self.group_readout(spikes.reshape(T * B, self.act_dim, self.dec_pop)).view(T, B, self.act_dim)
            raw = self.integrator(cur)[-1]                                        # potential after the last step
        functional.reset_net(self)
        return self.act_limit * torch.tanh(raw)


class Critic(nn.Module):
    def __init__(self, obs_dim: int, act_dim: int, hidden=(64, 64)):
        super().__init__()
        dims = (obs_dim + act_dim, *hidden, 1)
        layers = []
        for a, b in zip(dims[:-1], dims[1:]):
            layers += [nn.Linear(a, b), nn.ReLU()]
        self.net = nn.Sequential(*layers[:-1])

    def forward(self, obs, act):
        return self.net(torch.cat((obs, act), dim=-1)).squeeze(-1)


class ReplayBuffer:
    """Ring buffer with running observation statistics (Welford); sampled observations come out normalised and clipped."""

    def __init__(self, obs_dim: int, act_dim: int, size: int, clip: float = 5.0, noise_shape: Tuple[int, int] = (0, 0)):
        self.noise = np.zeros((size, *noise_shape), np.float32)
        self.obs, self.obs2 = np.zeros((size, obs_dim), np.float32), np.zeros((size, obs_dim), np.float32)
        self.act, self.rew, self.done = np.zeros((size, act_dim), np.float32), np.zeros(size, np.float32), np.zeros(size, np.float32)
        self.ptr = self.size = 0
        self.max_size, self.clip = size, clip
        self.mean, self.m2, self.count = np.zeros(obs_dim, np.float64), np.zeros(obs_dim, np.float64), 1e-4

    def store(self, o, a, r, o2, d, noise=None) -> None:
        i = self.ptr
        self.obs[i], self.act[i], self.rew[i], self.obs2[i], self.done[i] = o, a, r, o2, d
        if noise is not None and self.noise.shape[-1]:
            self.noise[i] = noise
        self.ptr, self.size = (i + 1) % self.max_size, min(self.size + 1, self.max_size)
        self.count += 1
        delta = o - self.mean
        self.mean += delta / self.count
        self.m2 += delta * (o - self.mean)

    def normalize(self, o: np.ndarray) -> np.ndarray:
        std = np.sqrt(self.m2 / self.count) + 1e-8
        return np.clip((o - self.mean) / std, -self.clip, self.clip).astype(np.float32)

    def sample(self, batch: int, device) -> Tuple[torch.Tensor, ...]:
        idx = np.random.randint(0, self.size, size=batch)
        t = lambda x: torch.as_tensor(x, device=device)
        return (t(self.normalize(self.obs[idx])), t(self.act[idx]), t(self.rew[idx]), t(self.normalize(self.obs2[idx])), t(self.done[idx]),
                t(self.noise[idx]))


class HybridTD3:
    def __init__(self, obs_dim, act_dim, act_limit, actor_kind="ilc", device="cpu", gamma=0.99, polyak=0.995, pi_lr=1e-3, q_lr=1e-3,
                 target_noise=0.2, noise_clip=0.5, policy_delay=2, **actor_kwargs):
        self.device, self.gamma, self.polyak, self.act_limit = torch.device(device), gamma, polyak, act_limit
        self.target_noise, self.noise_clip, self.policy_delay = target_noise, noise_clip, policy_delay
        self.actor = SpikingActor(obs_dim, act_dim, act_limit, actor_kind, **actor_kwargs).to(self.device)
        self.q1, self.q2 = Critic(obs_dim, act_dim).to(self.device), Critic(obs_dim, act_dim).to(self.device)
        self.targets = [copy.deepcopy(m).requires_grad_(False) for m in (self.actor, self.q1, self.q2)]
        self.targets[0].set_noise(False)                       # the target policy is evaluated without exploration noise
        self.pi_opt = torch.optim.Adam(self.actor.parameters(), lr=pi_lr)
        self.q_opt = torch.optim.Adam([*self.q1.parameters(), *self.q2.parameters()], lr=q_lr)
        self.updates = 0

    @torch.no_grad()
    def act(self, obs_norm: np.ndarray, noise: float = 0.0) -> np.ndarray:
        a = self.actor(torch.as_tensor(obs_norm, device=self.device).unsqueeze(0)).squeeze(0).cpu().numpy()
        if noise:
            a = a + noise * np.random.randn(*a.shape)
        return np.clip(a, -self.act_limit, self.act_limit).astype(np.float32)

    def update(self, batch) -> Tuple[float, float]:
        o, a, r, o2, d, cn = batch
        pi_t, q1_t, q2_t = self.targets
        with torch.no_grad():
            eps = (torch.randn_like(a) * self.target_noise).clamp(-self.noise_clip, self.noise_clip)
            a2 = (pi_t(o2) + eps).clamp(-self.act_limit, self.act_limit)
            backup = r + self.gamma * (1 - d) * torch.min(q1_t(o2, a2), q2_t(o2, a2))
        q_loss = F.mse_loss(self.q1(o, a), backup) + F.mse_loss(self.q2(o, a), backup)
        self.q_opt.zero_grad(set_to_none=True)
        q_loss.backward()
        self.q_opt.step()
        pi_loss = torch.zeros(())
        self.updates += 1
        if self.updates % self.policy_delay == 0:
            for p in self.q1.parameters():
                p.requires_grad_(False)
            if cn.shape[-1]:
                self.actor.load_colored_noise(cn)              # the policy is differentiated under the noise it acted with
            pi_loss = -self.q1(o, self.actor(o)).mean()
            self.actor.cancel_load()
            self.pi_opt.zero_grad(set_to_none=True)
            pi_loss.backward()
            self.pi_opt.step()
            for p in self.q1.parameters():
                p.requires_grad_(True)
            with torch.no_grad():
                for net, tgt in zip((self.actor, self.q1, self.q2), self.targets):
                    for p, pt in zip(net.parameters(), tgt.parameters()):
                        pt.mul_(self.polyak).add_((1 - self.polyak) * p)
        return float(q_loss.detach()), float(pi_loss.detach())


def _make_env(name: str, seed: int):
    if name != "builtin":
        for mod in ("gymnasium", "gym"):
            try:
                return __import__(mod).make(name)
            except Exception:
                continue
    return Pendulum(seed)


def _reset(env):
    out = env.reset()
    return np.asarray(out[0] if isinstance(out, tuple) else out, dtype=np.float32)


def _step(env, action):
    out = env.step(action)
    if len(out) == 5:
        o, r, term, trunc, _ = out
        return np.asarray(o, dtype=np.float32), float(r), bool(term or trunc)
    o, r, done = out[:3]
    return np.asarray(o, dtype=np.float32), float(r), bool(done)


def train(actor: str = "ilc", env_name: str = "builtin", steps: int = 4000, start_steps: int = 500, update_after: int = 500, batch_size: int = 64,
          act_noise: float = 0.1, seed: int = 0, device: str = "cpu", spike_ts: int = 5, log_every: int = 1000, quiet: bool = False):
    """Returns ``(agent, episode returns)``."""
    torch.manual_seed(seed)
    np.random.seed(seed)
    env = _make_env(env_name, seed)
    obs_dim = getattr(env, "obs_dim", None) or env.observation_space.shape[0]
    act_dim = getattr(env, "act_dim", None) or env.action_space.shape[0]
    act_limit = getattr(env, "act_limit", None) or float(env.action_space.high[0])
    agent = HybridTD3(obs_dim, act_dim, act_limit, actor, device, spike_ts=spike_ts)
    noisy = actor == "noisy"
    horizon = getattr(env, "max_steps", 1000) + 1
    buf = ReplayBuffer(obs_dim, act_dim, size=max(steps, 1000), noise_shape=(spike_ts, agent.actor.noise_length()) if noisy else (0, 0))
    if noisy:
        agent.actor.reset_noise(horizon)
    o, ep_ret, returns = _reset(env), 0.0, []
    for t in range(steps):
        a = np.random.uniform(-act_limit, act_limit, act_dim).astype(np.float32) if t < start_steps else agent.act(buf.normalize(o), act_noise)
        o2, r, done = _step(env, a)
        used = agent.actor.get_colored_noise().numpy() if (noisy and t >= start_steps) else None
        buf.store(o, a, r, o2, float(done and getattr(env, "t", 0) < getattr(env, "max_steps", 10 ** 9)), used)
        o, ep_ret = o2, ep_ret + r
        if done:
            returns.append(ep_ret)
            o, ep_ret = _reset(env), 0.0
            if noisy:
                agent.actor.reset_noise(horizon)
        if t >= update_after:
            agent.update(buf.sample(batch_size, agent.device))
        if not quiet and (t + 1) % log_every == 0 and returns:
            print(f"step {t + 1}: episodes {len(returns)}, mean return of the last 5 = {np.mean(returns[-5:]):.1f}")
    return agent, returns


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--actor", choices=["ilc", "noisy"], default="ilc")
    ap.add_argument("--env", default="builtin")
    ap.add_argument("--steps", type=int, default=4000)
    ap.add_argument("--spike-ts", type=int, default=5)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args()
    train(a.actor, a.env, a.steps, device=a.device, spike_ts=a.spike_ts, seed=a.seed)


if __name__ == "__main__":
    main()
