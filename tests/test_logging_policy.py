"""The logging lint (``utils/logging_policy.py``): each rule on small sources, and the package itself is clean."""
from pathlib import Path

from spikingjelly_b200.utils import logging_policy as LP


def _rules(src, **kw):
    return [v.rule for v in LP.check_source(src, **kw)]


def test_rules_fire_on_what_they_forbid():
    assert _rules("def f():\n    print('x')\n") == ["print"]
    assert _rules("import sys\ndef f():\n    sys.stderr.write('x')\n") == ["stream-write"]
    assert _rules("import logging\nlogging.info('x')\n") == ["root-logger"]
    assert _rules("import logging\nlogging.basicConfig()\n") == ["logging-setup"]
    assert _rules("import logging\nlog = logging.getLogger('x')\n") == ["private-logger"]
    assert _rules("from .logger import logger\nlogger.info(f'x={1}')\n") == ["eager-format"]
    assert _rules("from .logger import logger\nlogger.warning('a' + str(1))\n") == ["eager-format"]
    assert _rules("from .logger import logger\nlogger.debug('x=%s' % 1)\n") == ["eager-format"]
    assert _rules("from .logger import logger\nlogger.error('x={}'.format(1))\n") == ["eager-format"]
    assert _rules("def f(:\n") == ["syntax"]


def test_what_is_allowed():
    assert _rules("from .logger import logger\nlogger.info('x=%s', 1)\n") == []
    assert _rules("def main():\n    print('report')\n") == []                                  # command-line entry point
    assert _rules("if __name__ == '__main__':\n    print('report')\n") == []
    assert _rules("def check_manual_grad():\n    print('table')\n") == []                      # diagnostic helper
    assert _rules("print('x')\n", is_script=True) == []                                         # examples / benchmarks
    assert _rules("import logging\nlogger = logging.getLogger('pkg')\nlogger.addHandler(logging.NullHandler())\n",
                  is_logger_module=True) == []


def test_the_package_follows_its_own_policy():
    root = Path(LP.__file__).resolve().parents[1]
    found = LP.check_tree(root)
    assert not found, "\n".join(str(v) for v in found)
    assert LP.main([str(root)]) == 0
