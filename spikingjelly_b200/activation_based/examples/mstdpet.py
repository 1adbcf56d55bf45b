"""``mstdp.py`` with the eligibility-trace learner (``MSTDPETLearner``); kept as its own entry point because the reference has
``examples/mstdpet.py``."""
from .mstdp import main as _main


def main(argv=None) -> dict:
    return _main(["--eligibility-trace"] + list(argv or []))


if __name__ == "__main__":
    main()
