"""The example scripts run end to end on generated data (CPU, a couple of steps each)."""
import numpy as np
import pytest
import torch

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


def test_stdp_examples_run_and_match_closed_form():
    from spikingjelly_b200.activation_based.examples import mstdp, mstdpet, stdp_trace
    s = stdp_trace.main(["-T", "120"])
    assert s["post_spikes"] > 0 and abs(s["w_final"] - s["w_expected"]) < 1e-5
    s = mstdp.main(["-T", "120"])
    assert s["target_dw"] != 0.0 and s["other_dw"] < 1e-6
    s = mstdpet.main(["-T", "60"])
    assert s["other_dw"] < 1e-6


def test_recurrent_examples_run():
    from spikingjelly_b200.activation_based.examples import rsnn_sequential_fmnist, spiking_lstm_sequential_mnist
    for model in ("plain", "feedback"):
        s = rsnn_sequential_fmnist.main(["--model", model, "--synthetic", "--device", "cpu", "--max-steps", "3", "--hidden", "16", "-b", "16"])
        assert s["train_loss"] > 0
    s = spiking_lstm_sequential_mnist.main(["--synthetic", "--device", "cpu", "--max-steps", "2", "--hidden", "8", "-b", "8"])
    assert s["test_loss"] > 0


def test_dqn_examples_run_on_builtin_cartpole():
    from spikingjelly_b200.activation_based.examples import DQN_state, Spiking_DQN_state, _cartpole
    env = _cartpole.CartPole(0)
    s = _cartpole.reset_env(env)
    assert len(s) == 4
    steps = 0
    while True:                                  # always pushing one way tips the pole over well before the step cap
        s, r, over, fell = _cartpole.step_env(env, 1)
        steps += 1
        if over:
            break
    assert fell and 5 < steps < 100
    out = Spiking_DQN_state.main(["--episodes", "3", "--hidden", "16", "-T", "4", "--batch-size", "8", "--builtin-env"])
    assert out["best"] >= 1
    out = DQN_state.main(["--episodes", "3", "--hidden", "16", "--batch-size", "8", "--builtin-env"])
    assert out["best"] >= 1


def test_actor_critic_examples_run_on_builtin_cartpole():
    from spikingjelly_b200.activation_based.examples import A2C, PPO, Spiking_A2C, Spiking_PPO
    common = ["--episodes", "3", "--hidden", "16", "--builtin-env"]
    assert Spiking_A2C.main(common + ["-T", "4"])["best"] >= 1
    assert A2C.main(common)["best"] >= 1
    assert Spiking_PPO.main(common + ["-T", "4", "--horizon", "16", "--minibatch", "8", "--ppo-epochs", "1"])["best"] >= 1
    assert PPO.main(common + ["--horizon", "16", "--minibatch", "8", "--ppo-epochs", "1"])["best"] >= 1


def test_speechcommands_example_runs_on_synthetic_tones():
    from spikingjelly_b200.activation_based.examples import speechcommands as sc
    fb = sc.mel_filter_bank(257, 40, 20.0, 4000.0, 16000)
    assert fb.shape == (257, 40) and float(fb.min()) >= 0 and float(fb.sum(0).min()) > 0
    s = sc.main(["--synthetic", "--device", "cpu", "--max-steps", "4", "--channels", "8", "--n-mels", "16", "-b", "16", "--lr", "0.01"])
    assert s["train_loss"] > 0 and 0 <= s["test_acc"] <= 1


def test_spiking_lstm_text_example_learns_synthetic_languages():
    from spikingjelly_b200.activation_based.examples import spiking_lstm_text as ex
    assert ex.to_ascii("Ślusàrski") == "Slusarski" and ex.word_to_tensor("ab").shape == (2, 1, len(ex.LETTERS))
    s = ex.main(["--synthetic", "--steps", "150", "--hidden", "32"])
    assert s["last_loss"] < s["first_loss"] and s["test_acc"] > 0.4


def test_spiking_actor_td3_runs_with_both_actor_kinds():
    from spikingjelly_b200.activation_based.examples import spiking_actor_td3 as ex
    for kind in ("ilc", "noisy"):
        agent, returns = ex.train(kind, steps=260, start_steps=100, update_after=100, batch_size=8, quiet=True)
        assert agent.updates == 160 and len(returns) == 1 and returns[0] < 0
        act = agent.act(np.zeros(3, np.float32))
        assert act.shape == (1,) and abs(float(act[0])) <= 2.0
    assert ex.SpikingActor(3, 1, 2.0, "noisy").noise_length() == 2 * 64 + 2 * 64 + 2 * 10 + 1
    with pytest.raises(ValueError):
        ex.SpikingActor(3, 1, 2.0, "plain")


def test_dsqn_and_r11_examples_run():
    from spikingjelly_b200.activation_based.examples import DSQN
    from spikingjelly_b200.activation_based.examples import cifar10_r11_enabling_spikebased_backpropagation as r11
    net, rewards = DSQN.train(frames=160, T=2, size=8, batch_size=8, start=40, sync=50, quiet=True)
    assert len(rewards) == 160 // 7 and set(rewards) <= {1.0, -1.0}
    q = net(torch.zeros(2, 1, 8, 8))
    assert q.shape == (2, 3)
    _, hist = r11.main(["--synthetic", "-T", "12", "--width", "4", "--image-size", "16", "--samples", "32", "-b", "16", "--epochs", "3", "--device", "cpu",
                        "--lr", "0.05"])
    assert len(hist) == 3 and hist[-1][0] < hist[0][0]


def test_vector_environments():
    from functools import partial
    from spikingjelly_b200.activation_based.examples import _cartpole
    from spikingjelly_b200.activation_based.examples.common.multiprocessing_env import SerialVecEnv, SubprocVecEnv
    for cls in (SerialVecEnv, SubprocVecEnv):
        envs = cls([partial(_cartpole.CartPole, seed=i) for i in range(3)])
        obs = envs.reset()
        assert obs.shape == (3, 4) and len(envs) == 3
        for _ in range(30):
            obs, rew, done, info = envs.step([1, 0, 1])
        assert obs.shape == (3, 4) and rew.shape == (3,) and done.dtype == bool and len(info) == 3
        envs.close()


def test_memopt_example_loss_augmentation_and_callbacks():
    import numpy as np
    import torch.nn as nn
    from spikingjelly_b200.activation_based.examples.memopt import callbacks as C
    from spikingjelly_b200.activation_based.examples.memopt.data_module import CIFAR10DVSDataModule, CIFAR10DVSNDA, Cutout
    from spikingjelly_b200.activation_based.examples.memopt.loss import TETLoss, TMeanCrossEntropyLoss
    torch.manual_seed(0)
    y, label = torch.randn(5, 6, 10), torch.randint(0, 10, (6,))
    ce = nn.CrossEntropyLoss()
    want = 0.9 * sum(ce(y[t], label) for t in range(5)) / 5 + 0.1 * ((y - 1.5) ** 2).mean()
    assert torch.allclose(TETLoss(ce, mean=1.5, tet_lambda=0.1)(y, label), want, atol=1e-6)
    per_sample = TETLoss(nn.CrossEntropyLoss(reduction="sum"), tet_lambda=0.0)(y, label)        # non-mean criteria take the loop
    assert torch.allclose(per_sample, sum(nn.functional.cross_entropy(y[t], label, reduction="sum") for t in range(5)) / 5)
    assert torch.allclose(TMeanCrossEntropyLoss()(y, label), ce(y.mean(0), label))
    np.random.seed(0)
    img = torch.ones(3, 2, 16, 16)
    cut = Cutout(1, length=8)(img)
    assert 0 < (cut == 0).sum() <= 3 * 2 * 64 and cut.shape == img.shape
    assert CIFAR10DVSNDA(M=2, N=2)(torch.rand(4, 2, 32, 32)).shape == (4, 2, 32, 32)
    dm = CIFAR10DVSDataModule(None, T=3, batch_size=4, synthetic_samples=10, resolution=16)
    dm.prepare_data(), dm.setup()
    xb, yb = next(iter(dm.train_dataloader()))
    assert xb.shape == (4, 3, 2, 16, 16) and yb.shape == (4,) and len(dm.val_dataloader().dataset) == 2

    class T:
        is_global_zero, max_epochs, current_epoch, device = False, 1, 0, torch.device("cpu")
    t = C.GlobalMeanBatchTimeCallback(reset_per_epoch=False)
    for _ in range(3):
        t.on_train_batch_start(T, None, None, 0)
        t.on_train_batch_end(T, None, None, None, 0)
    t.on_train_epoch_end(T, None)
    assert t.totals["train"][1] == 3 and t.last["train"] >= 0
    t2 = C.GlobalMeanBatchTimeCallback()
    t2.load_state_dict(t.state_dict())
    assert t2.totals == t.totals
    s = C.SamplePerSecondCallback()
    s.on_train_epoch_start(T, None)
    s.on_train_batch_end(T, None, None, (torch.zeros(7, 2), torch.zeros(7)), 0)
    s.on_train_epoch_end(T, None)
    assert s.last["train"] > 0 and s.totals["train"] == [0.0, 0.0]


def test_memopt_example_trainer_runs_from_the_config(tmp_path):
    from spikingjelly_b200.activation_based.examples.memopt import train as M
    cfg = M.override({"a": {"b": 1}}, ["a.b=2.5", "a.c.d=true", "e=null"])
    assert cfg == {"a": {"b": 2.5, "c": {"d": True}}, "e": None}
    obj = M.instantiate({"class_path": "torch.nn.Linear", "init_args": {"in_features": 3, "out_features": 2}})
    assert isinstance(obj, torch.nn.Linear) and M.instantiate(5) == 5
    hist = M.main(["--device", "cpu", "--max-steps", "1", "--set", "data.synthetic=true", "data.T=2", "model.T=2", "data.batch_size=2",
                   "data.synthetic_samples=8", "trainer.max_epochs=1", "model.level=0", f"trainer.default_root_dir={tmp_path}"])
    assert len(hist) == 1 and (tmp_path / "metrics.csv").exists() and (tmp_path / "best.pt").exists()
    import pytest
    with pytest.raises(ValueError, match="differ"):
        M.main(["--device", "cpu", "--set", "data.T=3"])


def test_lava_and_lynxi_examples_run_up_to_the_vendor_step(tmp_path):
    from spikingjelly_b200.activation_based.examples import lava_mnist, lynxi_fmnist_inference
    stats = lava_mnist.main(["--synthetic", "--max-steps", "2", "-T", "4", "--channels", "4", "--device", "cpu", "--out-dir", str(tmp_path)])
    assert "train_loss" in stats and (tmp_path / "net.pt").exists()
    try:
        import lava.lib.dl.slayer  # noqa: F401
    except ImportError:
        assert stats["exported"] is False
    torch.manual_seed(0)
    res = lynxi_fmnist_inference.main(["--synthetic", "--channels", "8", "-T", "3", "-b", "4"])
    assert res["host_max_abs_diff"] < 1e-5
    try:
        import lynpy  # noqa: F401
    except ImportError:
        assert res["device"] is None


def test_conversion_examples_on_generated_data(tmp_path):
    """The ANN -> SNN example scripts end to end on generated data: the converted network reaches the source network's accuracy."""
    from spikingjelly_b200.activation_based.ann2snn.examples import cnn_mnist, imagenet_resnet18_ltb, imagenet_vit_sta, resnet18_cifar10
    out = cnn_mnist.main(["--synthetic", "--time-steps", "16", "--skip-mode-sweep", "--device", "cpu", "--max-eval-batches", "2", "--output", str(tmp_path / "cnn.json")])
    assert out["ann_accuracy"] > 0.8 and (tmp_path / "cnn.json").exists()
    assert all(r["snn_accuracy"] >= out["ann_accuracy"] - 0.1 for r in out["recipes"].values())
    out = resnet18_cifar10.main(["--synthetic", "--time-steps", "8", "--device", "cpu", "--max-eval-batches", "1"])
    assert 0.0 <= out["snn_accuracy"] <= 1.0 and "T=8" in out["curve"]
    out = imagenet_resnet18_ltb.main(["--synthetic", "--time-steps", "2", "--device", "cpu", "--delay-start", "auto", "--recipes", "ltb"])
    assert out["snn"]["ltb"]["delay_start"] == 17 and "T=2" in out["snn"]["ltb"]
    out = imagenet_vit_sta.main(["--synthetic", "--time-steps", "4", "--device", "cpu", "--modes", "equivalent"])
    assert out["snn"]["equivalent"]["top1"] == out["ann_top1"]                 # time-difference operators: exact after every step


def test_tempotron_example_learns_generated_digits():
    from spikingjelly_b200.timing_based.examples import tempotron_mnist
    history = tempotron_mnist.main(["--synthetic", "--epochs", "1", "-m", "4", "-T", "50", "--device", "cpu"])
    assert history[-1]["test_accuracy"] > 0.9
