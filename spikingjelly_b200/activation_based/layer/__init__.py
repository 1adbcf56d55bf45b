"""``layer`` namespace: step-mode aware layers."""
from .attention import *  # noqa: F401,F403
from .bn import *  # noqa: F401,F403
from .container import *  # noqa: F401,F403
from .dropout import *  # noqa: F401,F403
from .misc import *  # noqa: F401,F403
from .online_learning import *  # noqa: F401,F403
from .stateless import *  # noqa: F401,F403
