"""API-compatible counterpart of ``spikingjelly.activation_based``."""
