"""Import path of the reference's ``triton_kernel/neuron_kernel/lif.py``; the functions live in the package's ``__init__``."""
from . import *  # noqa: F401,F403
from . import __all__  # noqa: F401
from . import (LAST_BACKWARD_LOOP_MODE, LAST_FORWARD_LOOP_MODE, multistep_if_mixed_precision_forward,  # noqa: F401,E402
               multistep_if_mixed_precision_forward_with_plan, multistep_lif_mixed_precision_forward,
               multistep_lif_mixed_precision_forward_with_plan, multistep_plif_mixed_precision_forward,
               multistep_plif_mixed_precision_forward_with_plan)
