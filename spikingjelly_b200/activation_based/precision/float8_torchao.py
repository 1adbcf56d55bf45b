"""Import path of the reference's ``spikingjelly/activation_based/precision/float8_torchao.py``: the names below live in the ``precision`` package here."""
from . import Float8TorchAOPolicy  # noqa: F401

__all__ = ['Float8TorchAOPolicy']
