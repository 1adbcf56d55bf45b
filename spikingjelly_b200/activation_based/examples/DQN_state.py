"""``Spiking_DQN_state.py`` with the ordinary MLP Q-network (the reference's ``examples/DQN_state.py``)."""
from .Spiking_DQN_state import main as _main


def main(argv=None) -> dict:
    return _main(["--ann"] + list(argv or []))


if __name__ == "__main__":
    main()
