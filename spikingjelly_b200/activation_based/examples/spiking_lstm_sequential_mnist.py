"""Sequential MNIST with ``rnn.SpikingLSTM`` (the reference's ``examples/spiking_lstm_sequential_mnist.py``): the ``lstm`` model of
``rsnn_sequential_fmnist.py`` on MNIST."""
from .rsnn_sequential_fmnist import main as _main


def main(argv=None) -> dict:
    return _main(["--model", "lstm", "--dataset", "mnist"] + list(argv or []))


if __name__ == "__main__":
    main()
