"""Neuromorphic Intermediate Representation exchange (needs the optional ``nir`` / ``nirtorch`` packages at call time)."""
from .from_nir import *  # noqa: F401,F403
from .to_nir import *  # noqa: F401,F403
from ._spec import module_to_spec, spec_to_module  # noqa: F401
