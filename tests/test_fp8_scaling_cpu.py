"""Delayed and current fp8 scaling of ``ops/fp8.py`` on the CPU path (the CUDA kernels follow the same rotation of
three maxima; ``tests/test_fp8_gpu.py`` compares them with this path)."""
import torch

from spikingjelly_b200.ops import fp8


def test_first_call_scales_by_own_maximum_and_seeds_history():
    st = fp8.ScalingState()
    x = torch.randn(64, 128)
    q, qt, inv = fp8.quantize_with(x, st)
    assert qt is None and q.dtype == torch.float8_e4m3fn
    assert torch.allclose(inv, x.abs().amax().reshape(1) / fp8.E4M3_MAX)
    assert st.calls == 1 and torch.allclose(st.amax3[0], x.abs().amax())


def test_delayed_scale_is_the_previous_maximum():
    st = fp8.ScalingState()
    xs = [torch.randn(32, 64) * s for s in (1.0, 3.0, 0.5, 2.0, 7.0)]
    prev = None
    for k, x in enumerate(xs):
        q, _, inv = fp8.quantize_with(x, st)
        want = (x if prev is None else prev).abs().amax() / fp8.E4M3_MAX
        assert torch.allclose(inv, want.reshape(1)), k
        # values above the previous maximum saturate instead of overflowing
        assert torch.isfinite(q.float()).all()
        prev = x
    assert st.calls == len(xs)


def test_transposed_copy_matches():
    x = torch.randn(64, 128)
    q, qt, _ = fp8.quantize_with(x, None, e5m2=True, transpose=True)
    assert qt.shape == (128, 64) and qt.is_contiguous()
    assert torch.equal(qt.float(), q.float().t())


def test_linear_gradients_close_to_fp32_under_both_recipes():
    torch.manual_seed(0)
    x = (torch.rand(4, 32, 64) < 0.3).float().requires_grad_(True)
    w = (torch.randn(48, 64) * 0.1).requires_grad_(True)
    b = torch.zeros(48, requires_grad=True)
    gy = torch.randn(4, 32, 48)
    ref = torch.nn.functional.linear(x, w, b)
    gref = torch.autograd.grad(ref, (x, w, b), gy)
    for scaling in (None, fp8.LinearScaling()):
        for _ in range(3):                      # delayed scaling: the later calls run on history
            y = fp8.linear(x, w, b, scaling)
            g = torch.autograd.grad(y, (x, w, b), gy)
        assert torch.nn.functional.cosine_similarity(y.flatten(), ref.flatten(), dim=0) > 0.998
        for got, want in zip(g, gref):
            assert torch.nn.functional.cosine_similarity(got.flatten().float(), want.flatten(), dim=0) > 0.99


def test_policy_resolves_recipes():
    from spikingjelly_b200.activation_based.precision.float8_native import Float8Linear, Float8NativePolicy
    import torch.nn as nn
    for name, resolved in (("auto", "delayed"), ("delayed", "delayed"), ("current", "current"), ("mxfp8", "delayed")):
        pol = Float8NativePolicy(device_type="cpu", fp8_recipe=name)
        pol._resolved_recipe_name = None
        net = nn.Sequential(nn.Linear(32, 32), nn.ReLU(), nn.Linear(32, 16))

        class R:
            converted_modules, skipped_modules, converted_patterns = [], [], []
        out = pol._convert_modules(net, R)
        lins = [m for m in out.modules() if isinstance(m, Float8Linear)]
        assert len(lins) == 2 and all(m.fp8_recipe == resolved for m in lins)
        assert lins[0]._scaling().delayed == (resolved == "delayed")


def test_gradient_free_calls_reuse_the_quantised_weight():
    torch.manual_seed(0)
    w = torch.nn.Parameter(torch.randn(32, 64) * 0.1)
    x = torch.randn(16, 64)
    sc = fp8.LinearScaling()
    with torch.no_grad():
        y1 = fp8.linear(x, w, None, sc)
        first = sc._frozen
        y2 = fp8.linear(x, w, None, sc)
        assert sc._frozen is first
        w.mul_(2.0)                                   # an in-place update invalidates the cached bytes
        y3 = fp8.linear(x, w, None, sc)
        assert sc._frozen is not first
    ref = x @ w.detach().t()
    assert torch.nn.functional.cosine_similarity(y3.flatten(), ref.flatten(), dim=0) > 0.998
    assert torch.allclose(y3, 2 * y1, rtol=0.1, atol=0.05)
