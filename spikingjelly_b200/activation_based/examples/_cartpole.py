"""A dependency-free cart-pole (the classic Barto-Sutton-Anderson dynamics with the usual 12 degree / 2.4 m limits and a
500-step cap), so that the reinforcement-learning examples run where ``gym`` is not installed.  ``make_env`` returns a
``gymnasium`` / ``gym`` ``CartPole-v1`` when one of them can be imported and this class otherwise; both are driven through
:func:`reset_env` / :func:`step_env`, which hide the API differences."""
from __future__ import annotations

import math
import random
from typing import Tuple


class CartPole:
    gravity, masscart, masspole, length, force_mag, tau = 9.8, 1.0, 0.1, 0.5, 10.0, 0.02
    theta_limit, x_limit, max_steps = 12 * 2 * math.pi / 360, 2.4, 500
    n_states, n_actions = 4, 2

    def __init__(self, seed: int = 0):
        self.rng = random.Random(seed)
        self.state = (0.0, 0.0, 0.0, 0.0)
        self.steps = 0

    def reset(self):
        self.state = tuple(self.rng.uniform(-0.05, 0.05) for _ in range(4))
        self.steps = 0
        return list(self.state)

    def step(self, action: int):
        x, x_dot, th, th_dot = self.state
        force = self.force_mag if action == 1 else -self.force_mag
        total_mass, pml = self.masspole + self.masscart, self.masspole * self.length
        temp = (force + pml * th_dot ** 2 * math.sin(th)) / total_mass
        th_acc = (self.gravity * math.sin(th) - math.cos(th) * temp) / (self.length * (4.0 / 3.0 - self.masspole * math.cos(th) ** 2 / total_mass))
        x_acc = temp - pml * th_acc * math.cos(th) / total_mass
        x, x_dot = x + self.tau * x_dot, x_dot + self.tau * x_acc
        th, th_dot = th + self.tau * th_dot, th_dot + self.tau * th_acc
        self.state = (x, x_dot, th, th_dot)
        self.steps += 1
        fell = abs(x) > self.x_limit or abs(th) > self.theta_limit
        return list(self.state), 1.0, fell or self.steps >= self.max_steps, fell


def make_env(seed: int = 0, builtin: bool = False):
    if not builtin:
        for name in ("gymnasium", "gym"):
            try:
                mod = __import__(name)
                return mod.make("CartPole-v1")
            except Exception:
                continue
    return CartPole(seed)


def reset_env(env):
    out = env.reset()
    return list(out[0]) if isinstance(out, tuple) else list(out)


def step_env(env, action: int) -> Tuple[list, float, bool, bool]:
    """-> (state, reward, episode over, pole fell / cart left the track)"""
    out = env.step(action)
    if len(out) == 5:                       # gymnasium: obs, reward, terminated, truncated, info
        return list(out[0]), float(out[1]), bool(out[2] or out[3]), bool(out[2])
    if isinstance(env, CartPole):
        return out
    return list(out[0]), float(out[1]), bool(out[2]), bool(out[2])
