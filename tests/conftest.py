"""Test configuration.

* ``gpu`` marker: the test needs a CUDA device (run with ``-m gpu`` on a B200 box);
  everything else runs on CPU.
* ``reference`` fixture: the unmodified reference package, importable when it has been
  installed under ``baseline/_ref`` (tests that need it are skipped otherwise).
"""
import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
os.environ.setdefault("MASTER_ADDR", "127.0.0.1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def reference():
    ref_dir = ROOT / "baseline" / "_ref"
    if not (ref_dir / "spikingjelly").exists():
        pytest.skip("reference package not installed under baseline/_ref")
    sys.path.insert(0, str(ref_dir))
    try:
        import spikingjelly.activation_based as ab  # noqa: F401
        from spikingjelly.activation_based import functional, layer, neuron, surrogate, encoding
    except Exception as exc:  # pragma: no cover
        pytest.skip(f"reference package not importable: {exc}")
    finally:
        sys.path.remove(str(ref_dir))
    import types
    return types.SimpleNamespace(neuron=neuron, layer=layer, functional=functional, surrogate=surrogate,
                                 encoding=encoding)
