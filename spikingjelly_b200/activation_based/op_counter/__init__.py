"""Operation, memory-traffic and energy accounting of (spiking) networks."""
from .base import *  # noqa: F401,F403
from .compute_energy import *  # noqa: F401,F403
from .counters import *  # noqa: F401,F403
from ._sparse_memory import *  # noqa: F401,F403
from .neuron_state import *  # noqa: F401,F403
from .lemaire_addressing import *  # noqa: F401,F403
from .analytical_energy import *  # noqa: F401,F403
from .memory_residency import *  # noqa: F401,F403
from . import spikesim  # noqa: F401
from . import neuromc  # noqa: F401
from .neuromc import *  # noqa: F401,F403
from .spikesim import *  # noqa: F401,F403
