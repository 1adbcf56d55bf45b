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

# The reference splits three of these into packages (``distributed/pipeline/partition.py`` ...); here each is one module,
# so the sub-module paths resolve to that module.
for _pkg, _subs in (("pipeline", ("cifar10dvs_vgg", "memopt", "partition", "runtime", "spikformer")),
                    ("tensor_parallel", ("channel", "cifar10dvs_vgg", "debug", "linear", "spikformer", "state")),
                    ("adapters", ("base", "cifar10dvs_vgg", "spikformer"))):
    for _sub in _subs:
        sys.modules[f"{__name__}.{_pkg}.{_sub}"] = globals()[_pkg]
        if not hasattr(globals()[_pkg], _sub):          # ``import a.b.c as m`` reads the attribute c of a.b
            setattr(globals()[_pkg], _sub, globals()[_pkg])
