"""Bit pack / unpack kernel against the PyTorch formulation."""
import pytest
import torch

from spikingjelly_b200.ops import bitpack

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("n", [1, 7, 8, 127, 128, 4099, 1 << 20])
def test_pack_matches_torch_and_round_trips(dtype, n):
    torch.manual_seed(n)
    s = (torch.rand(n, device="cuda") > 0.7).to(dtype)
    packed = bitpack.bit_spike_compress(s)
    expect = bitpack._pack_torch((s != 0).reshape(-1))
    assert torch.equal(packed, expect)
    back = bitpack.bit_spike_decompress(packed, s.shape, dtype)
    assert back.dtype == dtype and torch.equal(back, s)


def test_unaligned_view_and_nd_shape():
    base = (torch.rand(3 * 5 * 11 + 1, device="cuda") > 0.5).float()
    s = base[1:].view(3, 5, 11)            # storage offset of 4 bytes: vector path must fall back
    packed = bitpack.bit_spike_compress(s)
    assert torch.equal(bitpack.bit_spike_decompress(packed, s.shape, torch.float32), s)


def test_checkpointed_block_on_gpu_matches_plain():
    import copy
    import torch.nn as nn
    from spikingjelly_b200.activation_based import functional, layer, memopt, neuron
    torch.manual_seed(0)
    plain = nn.Sequential(layer.Linear(64, 64, step_mode="m"), neuron.LIFNode(step_mode="m", backend="cuda")).cuda()
    boxed = memopt.GCContainer(memopt.BitSpikeCompressor(), *copy.deepcopy(plain))
    x = (torch.rand(4, 8, 64, device="cuda") > 0.5).float()
    y0 = plain(x); y0.sum().backward()
    y1 = boxed(x); y1.sum().backward()
    assert torch.equal(y0, y1)
    for p, q in zip(plain.parameters(), boxed.parameters()):
        assert torch.allclose(p.grad, q.grad, atol=1e-5)
