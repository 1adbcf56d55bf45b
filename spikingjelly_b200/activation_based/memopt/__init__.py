"""Memory optimisation: compressed-input gradient checkpointing and its automatic placement."""
from .checkpointing import *  # noqa: F401,F403
from .compress import *  # noqa: F401,F403
from .pipeline import *  # noqa: F401,F403
