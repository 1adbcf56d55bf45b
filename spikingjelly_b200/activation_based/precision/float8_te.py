"""Import path of the reference's ``spikingjelly/activation_based/precision/float8_te.py``: the names below live in the ``precision`` package here."""
from . import Float8TELayerNormLinearModule, Float8TELayerNormMLPModule, Float8TransformerEnginePolicy  # noqa: F401

__all__ = ['Float8TELayerNormLinearModule', 'Float8TELayerNormMLPModule', 'Float8TransformerEnginePolicy']
