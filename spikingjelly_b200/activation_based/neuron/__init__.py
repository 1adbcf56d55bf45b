"""``neuron`` namespace: spiking neuron modules."""
from .base_node import *  # noqa: F401,F403
from .integrate_and_fire import *  # noqa: F401,F403
from .lif import *  # noqa: F401,F403
from .lif_variants import *  # noqa: F401,F403
from .nonlinear_if import *  # noqa: F401,F403
from .psn import *  # noqa: F401,F403
from .training_variants import *  # noqa: F401,F403
from .conversion import *  # noqa: F401,F403
from .population import *  # noqa: F401,F403
from .flexsn import *  # noqa: F401,F403
