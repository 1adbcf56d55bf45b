"""Plot helpers: the data preparation always, the drawing where matplotlib exists."""
import numpy as np
import pytest
import torch

from spikingjelly_b200 import visualizing as V
from spikingjelly_b200.visualizing import _utils as U


def test_feature_map_grid_matches_loop():
    x = np.random.rand(6, 4, 5)
    g = U.feature_map_grid(x, 2, 3, space=2)
    ref = np.ones(((4 + 2) * 2, (5 + 2) * 3)) * x.max()
    k = 0
    for i in range(1, ref.shape[0], 6):
        for j in range(1, ref.shape[1], 7):
            ref[i:i + 4, j:j + 5] = x[k]
            k += 1
    assert np.array_equal(g, ref)
    with pytest.raises(ValueError):
        U.feature_map_grid(x, 2, 2, 1)


def test_spike_events_and_rates_and_conversion():
    s = torch.tensor([[1, 0], [0, 0], [1, 1.0]])
    ev = U.spike_events(U._to_numpy(s))
    assert ev[0].tolist() == [0, 2] and ev[1].tolist() == [2]
    assert np.allclose(U.firing_rates(s.numpy()), [[2 / 3], [1 / 3]])
    assert U._to_numpy(torch.ones(2, dtype=torch.bfloat16)).dtype == np.float32
    with pytest.raises(TypeError):
        U._to_numpy([1, 2])
    with pytest.raises(ValueError):
        V.plot_2d_heatmap(np.zeros(3), "t", "x", "y")
    with pytest.raises(ValueError):
        V.plot_one_neuron_v_s(np.zeros((2, 2)), np.zeros(2))


def test_drawing_with_matplotlib():
    pytest.importorskip("matplotlib")
    s = (torch.rand(20, 5) > 0.7).float()
    fig, ax = V.plot_1d_spikes(s, "spikes", "t", "neuron", dpi=50)
    assert len(fig.axes) == 2
    fig, ax = V.plot_2d_heatmap(torch.rand(20, 5), "v", "t", "neuron", x_max=10.0, dpi=50)
    assert ax.get_title() == "v"
    V.plot_2d_bar_in_3d(torch.rand(4, 3), "b", "x", "y", "z", dpi=50)
    V.plot_2d_feature_map(torch.rand(6, 4, 4), 2, 3, 2, "f", dpi=50)
    fig, a0, a1 = V.plot_one_neuron_v_s(np.random.rand(20), s[:, 0].numpy(), dpi=50)
    assert a1.get_xlabel() == "simulating step"
