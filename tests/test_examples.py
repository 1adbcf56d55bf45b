"""The example scripts run end to end on generated data (CPU, a couple of steps each)."""
from spikingjelly_b200.activation_based.examples import classify_dvsg, conv_fashion_mnist, flexsn_custom_neuron, lif_fc_mnist
from spikingjelly_b200.activation_based.examples.memopt import train_distributed


def test_lif_fc_mnist_learns_on_synthetic_data():
    stats = lif_fc_mnist.main(["--synthetic", "--device", "cpu", "--max-steps", "20", "-T", "8"])
    assert 0 < stats["train_loss"] < 0.5 and 0 <= stats["test_acc"] <= 1


def test_conv_and_dvsg_examples_run():
    s = conv_fashion_mnist.main(["--synthetic", "--device", "cpu", "--max-steps", "2", "--channels", "8", "-b", "8"])
    assert s["train_loss"] > 0
    s = classify_dvsg.main(["--synthetic", "--device", "cpu", "--max-steps", "1", "-T", "2", "--channels", "4", "-b", "2"])
    assert s["test_loss"] > 0


def test_flexsn_and_distributed_examples_run(capsys):
    flexsn_custom_neuron.main(["-N", "512", "-T", "3"])
    out = capsys.readouterr().out
    rates = [line.split("firing rate ")[1].split(",")[0] for line in out.splitlines() if "firing rate" in line]
    assert len(rates) == 2 and rates[0] == rates[1]
    train_distributed.main(["--synthetic", "--max-steps", "1", "--T", "2", "--batch-size", "2", "--resolution", "32"])
    assert "mode none" in capsys.readouterr().out
