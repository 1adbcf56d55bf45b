"""``activation_based.model``: the import path reference scripts use for the model zoo.  The
implementations live in :mod:`spikingjelly_b200.models`; every submodule is registered here under
its reference name, so that ``from ...activation_based.model import sew_resnet`` and
``import ...activation_based.model.sew_resnet`` both resolve to the same module object."""
import importlib
import sys

from ...models.spikformer import *  # noqa: F401,F403

_SUBMODULES = ("spikformer", "sew_resnet", "spiking_resnet", "spiking_vgg", "parametric_lif_net", "train_classify",
               "tv_ref_classify", "spiking_vggws_ottt", "snas_net", "spike_dhs", "train_imagenet_example",
               "train_flexsn_inductor_example")

for _name in _SUBMODULES:
    try:
        _mod = importlib.import_module(f"spikingjelly_b200.models.{_name}")
    except ModuleNotFoundError as _e:          # a model family that is not part of this build
        if _e.name != f"spikingjelly_b200.models.{_name}":
            raise
        continue
    sys.modules[f"{__name__}.{_name}"] = _mod
    globals()[_name] = _mod

# sub-modules of the torchvision-reference helpers, registered under this path as well: found through the package's
# ``__path__`` alone they would be loaded a second time under the alias name
for _name in ("presets", "sampler", "transforms", "utils"):
    _mod = importlib.import_module(f"spikingjelly_b200.models.tv_ref_classify.{_name}")
    sys.modules[f"{__name__}.tv_ref_classify.{_name}"] = _mod

from ...models.train_classify import Trainer  # noqa: E402,F401
