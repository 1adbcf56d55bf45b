"""When the fused model schedules may run and what they leave behind: they start from the reset state and do not keep
membrane potentials, so a second forward without ``reset_net`` must fail loudly instead of silently restarting; models
with SyncBatchNorm take the module path; a checkpointed segment updates batch-norm running statistics once."""
import pytest
import torch
import torch.nn as nn

pytestmark = pytest.mark.gpu


def _sew(dev):
    from spikingjelly_b200.activation_based import neuron, surrogate
    from spikingjelly_b200.models import sew_resnet
    net = sew_resnet.sew_resnet18(cnf="ADD", spiking_neuron=neuron.LIFNode, surrogate_function=surrogate.ATan(),
                                  detach_reset=True, backend="cuda", num_classes=11, in_channels=2).to(dev)
    from spikingjelly_b200.activation_based import functional
    functional.set_step_mode(net, "m")
    return net


def test_second_forward_without_reset_raises_and_reset_recovers():
    from spikingjelly_b200.activation_based import base, functional, neuron
    from spikingjelly_b200.models import _resnet_fused
    dev = torch.device("cuda")
    torch.manual_seed(0)
    net = _sew(dev)
    x = (torch.rand(2, 2, 2, 32, 32, device=dev) < 0.3).float()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        assert _resnet_fused.eligible(net, x)
        y0 = net(x)
        assert all(isinstance(m._memories["v"], base.ElidedState) for m in net.modules() if isinstance(m, neuron.BaseNode))
        assert not _resnet_fused.eligible(net, x)
        with pytest.raises(RuntimeError, match="reset_net"):
            net(x)
        functional.reset_net(net)
        assert _resnet_fused.eligible(net, x)
        y1 = net(x)
    assert torch.equal(y0, y1)


def test_sync_batchnorm_takes_the_module_path():
    from spikingjelly_b200.models import _resnet_fused
    dev = torch.device("cuda")
    net = nn.SyncBatchNorm.convert_sync_batchnorm(_sew(dev))
    x = torch.rand(2, 2, 2, 32, 32, device=dev)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        assert not _resnet_fused.eligible(net, x)


def test_checkpointed_fused_block_updates_running_stats_once():
    from spikingjelly_b200.activation_based import functional, layer, neuron, surrogate
    from spikingjelly_b200.activation_based.memopt import GCContainer, NullSpikeCompressor
    from spikingjelly_b200.models import _conv_fused

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.conv = layer.Conv2d(64, 64, 3, padding=1, bias=False, step_mode="m")
            self.bn = layer.BatchNorm2d(64, step_mode="m")
            self.sn = neuron.LIFNode(surrogate_function=surrogate.ATan(), detach_reset=True, step_mode="m", backend="cuda")

        def forward(self, x):
            assert _conv_fused.eligible(self.conv, self.bn, self.sn, x)
            return _conv_fused.conv_bn_lif(self.conv, self.bn, self.sn, x)

    dev = torch.device("cuda")
    torch.manual_seed(0)
    x = (torch.rand(2, 3, 64, 8, 8, device=dev) < 0.3).to(torch.bfloat16)
    plain, ckpt = Block().to(dev), Block().to(dev)
    ckpt.load_state_dict(plain.state_dict())
    wrapped = GCContainer(NullSpikeCompressor(), ckpt)
    xa, xb = x.clone().requires_grad_(), x.clone().requires_grad_()
    ya = plain(xa)
    yb = wrapped(xb)
    assert torch.equal(ya, yb)
    g = torch.randn_like(ya)
    ya.backward(g)
    yb.backward(g)
    assert int(plain.bn.num_batches_tracked) == 1 and int(ckpt.bn.num_batches_tracked) == 1
    torch.testing.assert_close(plain.bn.running_mean, ckpt.bn.running_mean)
    torch.testing.assert_close(plain.bn.running_var, ckpt.bn.running_var)
    torch.testing.assert_close(xa.grad.float(), xb.grad.float())
    torch.testing.assert_close(plain.conv.weight.grad, ckpt.conv.weight.grad)
    functional.reset_net(plain)
    functional.reset_net(ckpt)
