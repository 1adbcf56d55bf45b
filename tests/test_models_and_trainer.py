"""Model zoo shapes / state-dict layouts and one tiny end-to-end run of the classification trainer."""
import os

import pytest
import torch
import torch.nn as nn

from spikingjelly_b200.activation_based import functional, layer, neuron, surrogate
from spikingjelly_b200.activation_based.model import parametric_lif_net, sew_resnet, spiking_resnet, spiking_vgg
from spikingjelly_b200.models import train_classify


def test_alias_package_resolves_to_the_same_modules():
    import spikingjelly_b200.activation_based.model.sew_resnet as a
    import spikingjelly_b200.models.sew_resnet as b
    assert a is b and a is sew_resnet


@pytest.mark.parametrize("factory,kw", [(sew_resnet.sew_resnet18, dict(cnf="ADD")), (sew_resnet.sew_resnet50, dict(cnf="AND")),
                                        (spiking_resnet.spiking_resnet18, {}), (spiking_resnet.spiking_wide_resnet50_2, {})])
def test_resnets_keep_torchvision_state_dict_layout(factory, kw):
    import torchvision
    net = factory(spiking_neuron=neuron.IFNode, surrogate_function=surrogate.ATan(), detach_reset=True, **kw)
    tv = getattr(torchvision.models, factory.__name__.replace("sew_", "").replace("spiking_", ""))()
    assert list(net.state_dict().keys()) == list(tv.state_dict().keys())
    assert [v.shape for v in net.state_dict().values()] == [v.shape for v in tv.state_dict().values()]


def test_sew_resnet_event_input_and_step_modes():
    net = sew_resnet.sew_resnet18(spiking_neuron=neuron.LIFNode, surrogate_function=surrogate.ATan(), cnf="ADD",
                                  num_classes=11, in_channels=2)
    x = (torch.rand(3, 2, 2, 64, 64) < 0.1).float()
    net.eval()
    with torch.no_grad():
        y_s = torch.stack([net(x[t]) for t in range(3)])
        functional.reset_net(net)
        functional.set_step_mode(net, "m")
        y_m = net(x)
    assert y_m.shape == (3, 2, 11) and torch.allclose(y_s, y_m, atol=1e-5)
    with pytest.raises(NotImplementedError):
        sew_resnet.sew_function(x, x, "XOR")


def test_vgg_and_plif_nets():
    import torchvision
    net = spiking_vgg.spiking_vgg11_bn(spiking_neuron=neuron.IFNode, num_classes=10)
    assert list(net.state_dict().keys()) == list(torchvision.models.vgg11_bn(num_classes=10).state_dict().keys())
    x = torch.rand(2, 3, 32, 32)
    assert net(x).shape == (2, 10)
    functional.reset_net(net)
    single = spiking_vgg.sequential_forward(nn.Sequential(layer.Linear(4, 4), neuron.IFNode()), torch.rand(3, 2, 4))
    assert single.shape == (3, 2, 4)
    for cls, shape, out in [(parametric_lif_net.MNISTNet, (2, 1, 28, 28), 10), (parametric_lif_net.NMNISTNet, (2, 2, 32, 32), 10),
                            (parametric_lif_net.CIFAR10Net, (2, 3, 32, 32), 10), (parametric_lif_net.DVSGestureNet, (2, 2, 128, 128), 11)]:
        m = cls(8, neuron.ParametricLIFNode, surrogate_function=surrogate.ATan())
        assert m(torch.rand(shape)).shape == (2, out)


class _TinyTrainer(train_classify.Trainer):
    def load_data(self, args):
        import torchvision
        tf = torchvision.transforms.ToTensor()
        train = torchvision.datasets.FakeData(32, (3, 16, 16), 4, transform=tf)
        test = torchvision.datasets.FakeData(16, (3, 16, 16), 4, transform=tf, random_offset=7)
        train.classes = test.classes = list(range(4))
        return (train, test, *self._samplers(args, train, test))

    def load_model(self, args, num_classes):
        net = nn.Sequential(layer.Flatten(), layer.Linear(3 * 16 * 16, 32), neuron.LIFNode(surrogate_function=surrogate.ATan()),
                            layer.Linear(32, num_classes))
        functional.set_step_mode(net, "m")
        return net

    def preprocess_train_sample(self, args, x):
        return x.unsqueeze(0).repeat(args.T, 1, 1, 1, 1)

    preprocess_test_sample = preprocess_train_sample

    def process_model_output(self, args, y):
        return y.mean(0)

    def get_args_parser(self, add_help=True):
        p = super().get_args_parser(add_help)
        p.add_argument("--T", type=int, default=2)
        return p


def test_trainer_runs_resumes_and_checkpoints(tmp_path):
    torch.use_deterministic_algorithms(False)
    t = _TinyTrainer()
    common = ["--device", "cpu", "--epochs", "2", "-b", "8", "-j", "0", "--output-dir", str(tmp_path), "--opt", "adamw",
              "--lr", "0.01", "--lr-warmup-epochs", "1", "--disable-uda", "--model-ema", "--model-ema-steps", "1", "--T", "2"]
    args = t.get_args_parser().parse_args(common)
    t.main(args)
    pt_dir = os.path.join(str(tmp_path), "pt", t.get_tb_logdir_name(args))
    names = set(os.listdir(pt_dir))
    assert {"checkpoint_latest.pth", "checkpoint_1.pth", "checkpoint_max_test_acc1.pth"} <= names and "checkpoint_0.pth" not in names
    ckpt = torch.load(os.path.join(pt_dir, "checkpoint_latest.pth"), weights_only=False)
    assert ckpt["epoch"] == 1 and {"model", "optimizer", "lr_scheduler", "args", "max_test_acc1", "model_ema"} <= set(ckpt)
    assert not any("v" == k.split(".")[-1] for k in ckpt["model"])          # neuron state is never serialised
    latest = os.path.join(pt_dir, "checkpoint_latest.pth")
    args = t.get_args_parser().parse_args(common[:3] + ["3"] + common[4:] + ["--resume", latest])    # one more epoch
    t.main(args)
    pt_dir3 = os.path.join(str(tmp_path), "pt", t.get_tb_logdir_name(args))
    assert torch.load(os.path.join(pt_dir3, "checkpoint_latest.pth"), weights_only=False)["epoch"] == 2
    args = t.get_args_parser().parse_args(common + ["--resume", "latest", "--test-only"])
    t.main(args)
    torch.use_deterministic_algorithms(False)


def test_trainer_factories():
    t = train_classify.Trainer()
    args = t.get_args_parser().parse_args(["--opt", "sgd_nesterov", "--lr-scheduler", "step", "--lr-warmup-epochs", "0"])
    lin = nn.Linear(2, 2)
    opt = t.set_optimizer(args, lin.parameters())
    assert isinstance(opt, torch.optim.SGD) and opt.defaults["nesterov"]
    assert isinstance(t.set_lr_scheduler(args, opt), torch.optim.lr_scheduler.StepLR)
    args.opt = "lamb"
    with pytest.raises(RuntimeError, match="Invalid optimizer"):
        t.set_optimizer(args, lin.parameters())
    with pytest.raises(NotImplementedError):
        t.load_model(args, 10)


def test_ottt_vgg_family_builds_and_trains_online():
    from spikingjelly_b200.activation_based.model import spiking_vggws_ottt as O
    from spikingjelly_b200.activation_based import functional, layer
    net = O.ottt_spiking_vggws(num_classes=10)
    assert isinstance(net.features, layer.OTTTSequential) and sum(isinstance(m, layer.WSConv2d) for m in net.modules()) == 8
    x = torch.rand(2, 3, 32, 32)
    net.train()
    total = 0.0
    for _ in range(2):                                   # online: one backward per time step
        y = net(x)
        loss = (y - 1.0).square().mean()
        loss.backward()
        total += loss.item()
    functional.reset_net(net)
    assert y.shape == (2, 10) and net.classifier[2].weight.grad is not None and net.classifier[2].bias.grad.abs().sum() > 0 and total > 0
    full = O.ottt_spiking_vgg11_ws(num_classes=7)        # three-layer classifier with weight-standardised linears
    assert full(torch.rand(1, 3, 32, 32)).shape == (1, 7)
    assert [k for k in O.ottt_spiking_vgg16(num_classes=3).state_dict()][:2] == ["features.0.weight", "features.0.bias"]


@pytest.mark.gpu
@pytest.mark.parametrize("cnf", ["ADD", "AND", "IAND"])
def test_sew_resnet_fused_channels_last_schedule_matches_module_path(cnf):
    """Block by block (deep spiking stacks amplify single spike flips, so the whole net is only checked for statistics)."""
    from spikingjelly_b200.activation_based import functional, neuron, surrogate
    from spikingjelly_b200.models import _resnet_fused, sew_resnet
    from spikingjelly_b200.ops import counters
    torch.manual_seed(0)
    net = sew_resnet.sew_resnet18(num_classes=11, cnf=cnf, spiking_neuron=neuron.LIFNode, tau=2.0, detach_reset=True,
                                  surrogate_function=surrogate.ATan(), in_channels=2).cuda()
    functional.set_step_mode(net, "m")
    functional.set_backend(net, "cuda", instance=neuron.LIFNode)
    T, B = 4, 4
    rel = lambda a, b: ((a - b).norm() / (b.norm() + 1e-12)).item()
    for blk, cin, hw in ((net.layer1[0], 64, 16), (net.layer2[0], 64, 16), (net.layer4[1], 512, 4)):
        x = (torch.rand(T, B, cin, hw, hw, device="cuda") < 0.3).float()
        outs, grads = [], []
        for fused in (True, False):
            blk.zero_grad(set_to_none=True)
            functional.reset_net(blk)
            xi = x.clone().requires_grad_(True)
            with torch.autocast("cuda", dtype=torch.bfloat16):
                if fused:
                    h = xi.flatten(0, 1).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
                    o = _resnet_fused._block(blk, h, T)
                    o = o.reshape(T, B, *o.shape[1:])
                else:
                    o = blk(xi)
            o.float().mul(torch.linspace(0.5, 1.5, o.shape[2], device="cuda").view(1, 1, -1, 1, 1)).sum().backward()
            outs.append(o.detach().float())
            grads.append((xi.grad.clone(), blk.conv1.weight.grad.float().clone()))
        functional.reset_net(blk)
        assert outs[0].shape == outs[1].shape and (outs[0] != outs[1]).float().mean() < 0.02, type(blk).__name__
        tol = 0.2 if cnf == "ADD" else 0.45          # products of spike trains amplify single flips in the gradient
        assert rel(grads[0][0], grads[1][0]) < tol and rel(grads[0][1], grads[1][1]) < tol
    x = (torch.rand(T, B, 2, 64, 64, device="cuda") < 0.3).float()
    stats = {}
    for name in ("fused", "module"):
        functional.reset_net(net)
        before = counters.by_name().get("bn_lif_forward", 0)
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            assert _resnet_fused.eligible(net, x)
            out = net(x) if name == "fused" else net._forward_impl(x)
        used = counters.by_name().get("bn_lif_forward", 0) - before
        assert (used == 20) if name == "fused" else (used == 0)          # 17 conv stages + 3 down-sampling shortcuts
        stats[name] = out.float()
    functional.reset_net(net)
    assert stats["fused"].shape == (T, B, 11) and torch.isfinite(stats["fused"]).all()
    assert abs(stats["fused"].std().item() - stats["module"].std().item()) < 0.5 * stats["module"].std().item() + 1e-3


@pytest.mark.gpu
def test_vgg_fused_conv_bn_lif_matches_module_path():
    """CIFAR10-DVS VGG blocks under bf16 autocast: fused channels-last schedule against the modules' own forward, block by
    block (spike mismatch from 16-bit rounding stays small; gradients agree within the tolerance of bf16 accumulation)."""
    from spikingjelly_b200 import ops
    from spikingjelly_b200.activation_based import functional
    from spikingjelly_b200.activation_based.examples.memopt.models import CIFAR10DVSVGG
    from spikingjelly_b200.models import _conv_fused
    ops.require()
    torch.manual_seed(0)
    net = CIFAR10DVSVGG(dropout=0.0, backend="cuda").cuda().train()
    x = (torch.rand(4, 2, 6, 2, 48, 48, device="cuda") < 0.3).float()[0].transpose(0, 1).contiguous()   # [T=6, N=2, ...] built from [N, T]
    x = x.reshape(6, 2, 2, 48, 48)
    blk = net.features[1]                       # 64 -> 128 channels, spikes in
    s_in = (torch.rand(6, 2, 64, 48, 48, device="cuda") < 0.2).float().requires_grad_(True)
    conv, bn = blk.proj_bn[-2], blk.proj_bn[-1]
    with torch.autocast("cuda", dtype=torch.bfloat16):
        assert _conv_fused.eligible(conv, bn, blk.neuron, s_in)
        out_f = blk(s_in)
        g = torch.randn_like(out_f)
        out_f.backward(g)
    gf, gw_f = s_in.grad.clone(), conv.weight.grad.clone()
    s_in.grad = None
    net.zero_grad()
    functional.reset_net(net)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out_m = blk.neuron(blk.proj_bn(s_in))     # the modules' own path
        out_m.backward(g.to(out_m.dtype))
    assert out_f.shape == out_m.shape
    mismatch = (out_f.float() != out_m.float()).float().mean().item()
    assert mismatch < 0.02
    rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm()).item()    # noqa: E731
    assert rel(gw_f, conv.weight.grad) < 0.25 and rel(gf, s_in.grad) < 0.25
    functional.reset_net(net)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = net(torch.rand(2, 6, 2, 48, 48, device="cuda"))
    assert y.shape == (6, 2, 10) and torch.isfinite(y.float()).all()


@pytest.mark.gpu
def test_spiking_vgg_fused_triples_under_autocast():
    from spikingjelly_b200 import ops
    from spikingjelly_b200.activation_based import functional, neuron, surrogate
    from spikingjelly_b200.models import spiking_vgg
    from spikingjelly_b200.ops import counters
    ops.require()
    torch.manual_seed(0)
    net = spiking_vgg.spiking_vgg11_bn(spiking_neuron=neuron.LIFNode, surrogate_function=surrogate.ATan(), detach_reset=True,
                                       num_classes=10).cuda().train()
    functional.set_step_mode(net, "m")
    functional.set_backend(net, "cuda", instance=neuron.LIFNode)
    x = torch.rand(2, 2, 3, 64, 64, device="cuda")
    counters.reset()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = net(x)
        y.float().mean().backward()
    assert y.shape == (2, 2, 10) and torch.isfinite(y.float()).all()
    assert counters.by_name().get("bn_lif_forward", 0) == 8          # the eight convolution stages of VGG-11 ran fused
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in net.features.parameters())
    functional.reset_net(net)


def test_example_trainers_build_their_models_and_shapes():
    """``SResNetTrainer`` / ``FlexSNTrainer``: argument parsing, model construction, sample repetition and rate read-out."""
    from spikingjelly_b200.activation_based.model import train_flexsn_inductor_example as F, train_imagenet_example as R
    from spikingjelly_b200.models.train_imagenet_example import SResNetTrainer
    assert R.SResNetTrainer is SResNetTrainer
    t = R.SResNetTrainer()
    args = t.get_args_parser().parse_args(["--T", "3", "--model", "spiking_resnet18", "--cupy"])
    assert t.get_tb_logdir_name(args).endswith("_T3")
    net = t.load_model(args, 7)
    x = t.preprocess_train_sample(args, torch.rand(2, 3, 32, 32))
    assert x.shape == (3, 2, 3, 32, 32)
    with torch.no_grad():
        y = t.process_model_output(args, net(x))
    assert y.shape == (2, 7)
    args.model = "resnet18"
    with pytest.raises(ValueError, match="args.model should be one of"):
        t.load_model(args, 7)
    f = F.FlexSNTrainer()
    fargs = f.get_args_parser().parse_args(["--T", "2", "--model", "spiking_vgg11_bn", "--surrogate-alpha", "2.0"])
    assert "flexsn_cuda_sa2.0" in f.get_tb_logdir_name(fargs)
    vgg = f.load_model(fargs, 5)
    flex = [m for m in vgg.modules() if isinstance(m, neuron.FlexSN)]
    assert len(flex) == 10 and flex[0].step_mode == "m"
    with torch.no_grad():
        out = f.process_model_output(fargs, vgg(f.preprocess_test_sample(fargs, torch.rand(1, 3, 32, 32))))
    assert out.shape == (1, 5)
