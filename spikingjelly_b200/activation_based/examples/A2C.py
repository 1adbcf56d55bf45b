"""``Spiking_A2C.py`` run with ``--ann`` (the reference's ``examples/A2C.py``)."""
from .Spiking_A2C import main as _main


def main(argv=None) -> dict:
    return _main(['--ann'] + list(argv or []))


if __name__ == "__main__":
    main()
