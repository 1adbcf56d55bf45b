"""Model zoo."""
from . import spikformer  # noqa: F401
from .spikformer import *  # noqa: F401,F403
