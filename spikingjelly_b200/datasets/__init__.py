"""Neuromorphic and audio datasets.  ``spikingjelly_b200.datasets.<module>.<Class>`` mirrors the reference layout;
the common helpers are re-exported here (``spikingjelly/datasets/__init__.py``)."""
from .base import *  # noqa: F401,F403
from .transform import *  # noqa: F401,F403
from .utils import *  # noqa: F401,F403
from . import (asl_dvs, bullying10k, cifar10_dvs, dvs128_gesture, dvs_lip, es_imagenet, hardvs, n_caltech101, n_mnist,  # noqa: F401
               nav_gesture, shd, speechcommands)
from .asl_dvs import *  # noqa: F401,F403,E402
from .bullying10k import *  # noqa: F401,F403,E402
from .cifar10_dvs import *  # noqa: F401,F403,E402
from .dvs_lip import *  # noqa: F401,F403,E402
from .dvs128_gesture import *  # noqa: F401,F403,E402
from .es_imagenet import *  # noqa: F401,F403,E402
from .hardvs import *  # noqa: F401,F403,E402
from .n_caltech101 import *  # noqa: F401,F403,E402
from .n_mnist import *  # noqa: F401,F403,E402
from .nav_gesture import *  # noqa: F401,F403,E402
from .shd import *  # noqa: F401,F403,E402
from .speechcommands import *  # noqa: F401,F403,E402
