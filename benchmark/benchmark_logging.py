#!/usr/bin/env python
"""Cost of a logging call of the package logger when it is filtered by level, sent to a null handler, formatted, or
filtered by the handler (counterpart of the reference's ``benchmark/benchmark_logging.py``; ``--impl reference`` measures the
reference's logger).  Hot paths guard their log calls with ``logger.isEnabledFor`` (``utils/logging_policy.py``), so the
first row is what an unlogged training step pays per call site.

    python benchmark/benchmark_logging.py [--calls 1000000] [--impl ours|reference]
"""
import argparse
import json
import logging
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))
import _arms  # noqa: E402


class _Formatting(logging.Handler):
    def __init__(self):
        super().__init__()
        self.setFormatter(logging.Formatter("%(levelname)s %(message)s"))

    def emit(self, record):
        self.format(record)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--calls", type=int, default=1_000_000)
    a = ap.parse_args()
    if a.impl == "ours":
        sys.path.insert(0, str(_arms.ROOT))
        from spikingjelly_b200.logger import logger
    else:
        sys.path.insert(0, str(_arms.REF_DIR))
        from spikingjelly.logger import logger
    logger.propagate = False
    t0 = time.perf_counter()
    for _ in range(a.calls):
        pass
    base = time.perf_counter() - t0
    rows = {"empty_loop": base / a.calls * 1e9}
    for name, level, handler, handler_level in (("logger_filtered", logging.WARNING, None, None), ("null_handler", logging.INFO, logging.NullHandler(), logging.INFO),
                                                ("formatted_handler", logging.INFO, _Formatting(), logging.INFO),
                                                ("handler_filtered", logging.INFO, logging.NullHandler(), logging.WARNING),
                                                ("guarded_by_isEnabledFor", logging.WARNING, None, None)):
        logger.handlers.clear()
        logger.setLevel(level)
        if handler is not None:
            handler.setLevel(handler_level)
            logger.addHandler(handler)
        t0 = time.perf_counter()
        if name == "guarded_by_isEnabledFor":
            for i in range(a.calls):
                if logger.isEnabledFor(logging.INFO):
                    logger.info("benchmark index=%s", i)
        else:
            for i in range(a.calls):
                logger.info("benchmark index=%s", i)
        rows[name] = (time.perf_counter() - t0) / a.calls * 1e9
    print(json.dumps({"impl": a.impl, "calls": a.calls, "ns_per_call": {k: round(v, 1) for k, v in rows.items()}}))


if __name__ == "__main__":
    main()
