"""``functional`` namespace: stateless ops and whole-network helpers."""
from .forward import *  # noqa: F401,F403
from .layer import *  # noqa: F401,F403
from .learning import *  # noqa: F401,F403
from .loss import *  # noqa: F401,F403
from .misc import *  # noqa: F401,F403
from .net_config import *  # noqa: F401,F403
from .neuron import *  # noqa: F401,F403
from .online_learning import *  # noqa: F401,F403
# conv_bn_fusion is imported on demand (it needs ``layer``).
