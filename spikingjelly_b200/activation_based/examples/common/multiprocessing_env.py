"""Vectorised environments for the actor-critic examples: ``SubprocVecEnv([make_env] * n)`` steps ``n`` environments in
worker processes behind one batched ``reset`` / ``step`` (role of the reference's ``examples/common/multiprocessing_env.py``,
there a copy of the OpenAI-baselines vector environment).  ``SerialVecEnv`` has the same interface in one process, for
tests and for environments that cannot be pickled.  Both accept classic (4-tuple) and gymnasium-style (5-tuple) ``step``
results and reset an environment automatically when its episode ends."""
from __future__ import annotations

import multiprocessing as mp
from typing import Callable, List, Sequence

import numpy as np

__all__ = ["VecEnv", "SerialVecEnv", "SubprocVecEnv"]


def _reset(env):
    out = env.reset()
    return out[0] if isinstance(out, tuple) and len(out) == 2 and isinstance(out[1], dict) else out


def _step(env, action):
    out = env.step(action)
    if len(out) == 5:
        ob, reward, terminated, truncated, info = out
        done = bool(terminated or truncated)
    else:
        ob, reward, done = out[:3]
        info = out[3] if len(out) > 3 else {}
    if done:
        ob = _reset(env)
    return ob, float(reward), bool(done), info


class VecEnv:
    """``reset() -> obs [n, ...]``; ``step(actions) -> (obs [n, ...], rewards [n], dones [n], infos)``; ``close()``."""
    num_envs: int

    def reset(self):
        raise NotImplementedError

    def step_async(self, actions) -> None:
        raise NotImplementedError

    def step_wait(self):
        raise NotImplementedError

    def step(self, actions):
        self.step_async(actions)
        return self.step_wait()

    def close(self) -> None:
        pass

    def __len__(self) -> int:
        return self.num_envs


class SerialVecEnv(VecEnv):
    def __init__(self, env_fns: Sequence[Callable]):
        self.envs = [fn() for fn in env_fns]
        self.num_envs = len(self.envs)
        self._pending = None

    def reset(self):
        return np.stack([np.asarray(_reset(e), dtype=np.float32) for e in self.envs])

    def step_async(self, actions) -> None:
        self._pending = actions

    def step_wait(self):
        results = [_step(e, a) for e, a in zip(self.envs, self._pending)]
        obs, rews, dones, infos = zip(*results)
        return np.stack([np.asarray(o, dtype=np.float32) for o in obs]), np.asarray(rews, np.float32), np.asarray(dones), list(infos)


def _worker(remote, parent_remote, env_fn) -> None:
    parent_remote.close()
    env = env_fn()
    try:
        while True:
            cmd, data = remote.recv()
            if cmd == "step":
                remote.send(_step(env, data))
            elif cmd == "reset":
                remote.send(_reset(env))
            elif cmd == "close":
                break
            else:
                raise NotImplementedError(cmd)
    finally:
        remote.close()


class SubprocVecEnv(VecEnv):
    """One worker process per environment.  ``env_fns`` must be picklable callables (module-level functions or
    ``functools.partial`` objects) under the ``spawn`` start method; ``start_method`` defaults to ``fork`` where available."""

    def __init__(self, env_fns: Sequence[Callable], start_method: str = None):
        ctx = mp.get_context(start_method or ("fork" if "fork" in mp.get_all_start_methods() else "spawn"))
        self.num_envs = len(env_fns)
        self.remotes, work_remotes = zip(*[ctx.Pipe() for _ in range(self.num_envs)])
        self.procs: List = [ctx.Process(target=_worker, args=(w, r, fn), daemon=True) for w, r, fn in zip(work_remotes, self.remotes, env_fns)]
        for p in self.procs:
            p.start()
        for w in work_remotes:
            w.close()
        self.waiting = self.closed = False

    def reset(self):
        for r in self.remotes:
            r.send(("reset", None))
        return np.stack([np.asarray(r.recv(), dtype=np.float32) for r in self.remotes])

    def step_async(self, actions) -> None:
        for r, a in zip(self.remotes, actions):
            r.send(("step", a))
        self.waiting = True

    def step_wait(self):
        results = [r.recv() for r in self.remotes]
        self.waiting = False
        obs, rews, dones, infos = zip(*results)
        return np.stack([np.asarray(o, dtype=np.float32) for o in obs]), np.asarray(rews, np.float32), np.asarray(dones), list(infos)

    def close(self) -> None:
        if self.closed:
            return
        if self.waiting:
            for r in self.remotes:
                r.recv()
        for r in self.remotes:
            r.send(("close", None))
        for p in self.procs:
            p.join(timeout=5)
        self.closed = True
