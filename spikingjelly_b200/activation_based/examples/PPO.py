"""``Spiking_A2C.py`` run with ``--ann --ppo`` (the reference's ``examples/PPO.py``)."""
from .Spiking_A2C import main as _main


def main(argv=None) -> dict:
    return _main(['--ann', '--ppo'] + list(argv or []))


if __name__ == "__main__":
    main()
