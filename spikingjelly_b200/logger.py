"""Package logger.  Library code logs through ``logger`` only; the application
decides about handlers and levels (a ``NullHandler`` keeps the library silent by
default).  Parity: ``spikingjelly/logger.py:36-42``.
"""
import logging

logger: logging.Logger = logging.getLogger("spikingjelly_b200")
logger.addHandler(logging.NullHandler())

__all__ = ["logger"]
