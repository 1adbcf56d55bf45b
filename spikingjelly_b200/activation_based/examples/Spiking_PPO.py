"""``Spiking_A2C.py`` run with ``--ppo`` (the reference's ``examples/Spiking_PPO.py``)."""
from .Spiking_A2C import main as _main


def main(argv=None) -> dict:
    return _main(['--ppo'] + list(argv or []))


if __name__ == "__main__":
    main()
