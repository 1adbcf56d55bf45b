"""Import path of the reference's ``triton_kernel/neuron_kernel/integrate_and_fire.py``; the functions live in the package's ``__init__``."""
from . import *  # noqa: F401,F403
from . import __all__  # noqa: F401
