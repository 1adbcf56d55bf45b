"""``activation_based.distributed``: the import path of the reference's distributed package.  The
implementation lives in :mod:`spikingjelly_b200.parallel`; its submodules are registered here under
the reference's names (``distributed.api``, ``distributed.planner``, ``distributed.tensor_parallel`` ...)."""
import importlib
import sys

from ...parallel import *  # noqa: F401,F403
from ...parallel import __all__  # noqa: F401

for _name in ("api", "analysis", "config", "data_parallel", "execution", "fsdp", "mesh", "metrics", "optimizer", "pipeline", "planner",
              "runtime", "tensor_parallel", "topology", "adapters", "comm"):
    _mod = importlib.import_module(f"spikingjelly_b200.parallel.{_name}")
    sys.modules[f"{__name__}.{_name}"] = _mod
    globals()[_name] = _mod
