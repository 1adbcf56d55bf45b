"""fp8 tensor-core GEMM, quantisation kernels and the differentiable fp8 linear."""
import pytest
import torch

from spikingjelly_b200.ops import fp8

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("e5m2", [False, True])
def test_quantize_matches_reference_formulation(dtype, e5m2):
    torch.manual_seed(0)
    x = (torch.randn(1000, 37, device="cuda") * 3).to(dtype)
    q, inv = fp8.quantize(x, e5m2)
    fmax = fp8.E5M2_MAX if e5m2 else fp8.E4M3_MAX
    scale = fmax / x.float().abs().max()
    ref = (x.float() * scale).clamp(-fmax, fmax).to(q.dtype)
    assert torch.allclose(inv, (1 / scale).reshape(1), rtol=1e-6)
    assert torch.equal(q.view(torch.uint8), ref.view(torch.uint8))
    zero_q, zero_inv = fp8.quantize(torch.zeros(64, device="cuda", dtype=dtype), e5m2)
    assert float(zero_inv) == 1.0 and not zero_q.float().any()


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (300, 512, 256), (25088, 512, 512), (25088, 2048, 512), (77, 136, 2064),
                                   (64, 64, 8192)])
@pytest.mark.parametrize("fmt", [torch.float8_e4m3fn, torch.float8_e5m2])
def test_gemm_fp8_equals_fp32_matmul_of_the_same_fp8_values(M, N, K, fmt):
    torch.manual_seed(M + N + K)
    a = (torch.randn(M, K, device="cuda")).to(fmt)
    b = (torch.randn(N, K, device="cuda")).to(fmt)
    alpha = torch.tensor([0.37], device="cuda")
    got = fp8.matmul_nt(a, b, alpha, out_f32=True)
    ref = (a.float() @ b.float().t()) * 0.37
    # products of fp8 values are exact in fp32; only the accumulation order differs
    assert torch.allclose(got, ref, rtol=1e-4, atol=1e-3 * K ** 0.5)
    got16 = fp8.matmul_nt(a, b, alpha)
    assert got16.dtype == torch.bfloat16 and torch.allclose(got16.float(), ref, rtol=1e-2, atol=2e-2 * K ** 0.5)
    from spikingjelly_b200.ops import gemm
    gemm.check_status(a)


def test_spike_inputs_are_exact():
    torch.manual_seed(1)
    s = (torch.rand(512, 256, device="cuda") > 0.8).to(torch.bfloat16)
    w = torch.randn(128, 256, device="cuda", dtype=torch.bfloat16) * 0.05
    sq, si = fp8.quantize(s)
    assert float(si) == pytest.approx(1 / 448.0) and torch.equal(fp8.dequantize(sq, si), s)
    wq, wi = fp8.quantize(w)
    y = fp8.matmul_nt(sq, wq, si * wi, out_f32=True)
    ref = s.float() @ fp8.dequantize(wq, wi, torch.float32).t()
    assert torch.allclose(y, ref, rtol=1e-4, atol=1e-4)


def test_fp8_linear_forward_backward_close_to_bf16():
    torch.manual_seed(2)
    x = torch.randn(4, 196, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(1024, 512, device="cuda") * 0.03).requires_grad_(True)
    b = torch.randn(1024, device="cuda").requires_grad_(True)
    y = fp8.linear(x, w, b)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br = x.detach().float().requires_grad_(True), w.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(g.float())
    cos = lambda a, b_: torch.nn.functional.cosine_similarity(a.flatten().float(), b_.flatten().float(), dim=0).item()
    rel = lambda a, b_: ((a.float() - b_.float()).norm() / b_.float().norm()).item()
    for got, ref in ((y, yr), (x.grad, xr.grad), (w.grad, wr.grad), (b.grad, br.grad)):
        assert cos(got, ref) > 0.99 and rel(got, ref) < 0.12, (cos(got, ref), rel(got, ref))


def test_fp8_policy_trains_a_spiking_mlp():
    import torch.nn as nn
    from spikingjelly_b200.activation_based import functional, layer, neuron, precision, surrogate
    torch.manual_seed(0)
    net = nn.Sequential(layer.Linear(256, 512), neuron.LIFNode(surrogate_function=surrogate.ATan(), backend="cuda"),
                        layer.Linear(512, 512), neuron.LIFNode(surrogate_function=surrogate.ATan(), backend="cuda"),
                        layer.Linear(512, 16)).cuda()
    functional.set_step_mode(net, "m")
    art = precision.prepare_model_for_precision(net, "cuda", {"mode": "fp8", "strictness": "strict"})
    assert art.effective_config.mode == "fp8" and art.scaler is None
    assert art.describe()["capability_report"]["native_fp8_available"] is True
    assert len(art.describe()["conversion_report"]["converted_modules"]) == 3
    opt = torch.optim.Adam(art.model.parameters(), lr=3e-3)
    x = torch.rand(4, 64, 256, device="cuda")
    target = torch.randint(0, 16, (64,), device="cuda")
    losses = []
    for _ in range(60):
        with art.autocast_context():
            out = art.model(x).float().mean(0)
        loss = torch.nn.functional.cross_entropy(out, target)
        opt.zero_grad()
        art.backward(loss, opt)
        functional.reset_net(art.model)
        losses.append(float(loss))
    assert all(l == l for l in losses) and min(losses[-5:]) < losses[0], losses


@pytest.mark.parametrize("e5m2", [False, True])
@pytest.mark.parametrize("shape,transpose", [((1000, 40), False), ((128, 256), True), ((192, 128), True), ((64, 384), True)])
def test_delayed_and_transposing_kernels_follow_the_cpu_formulation(e5m2, shape, transpose):
    torch.manual_seed(3)
    dev_state = fp8.ScalingState()
    cpu_state = fp8.ScalingState()
    for k, s in enumerate((1.0, 2.5, 0.3, 4.0, 1.0)):
        x = (torch.randn(*shape, device="cuda") * s).to(torch.bfloat16)
        used = None if dev_state.calls == 0 else dev_state.amax3[(dev_state.calls + 2) % 3].clone()
        q, qt, inv = fp8.quantize_with(x, dev_state, e5m2=e5m2, transpose=transpose)
        # scale and history follow the CPU formulation; the bytes equal the same formula evaluated by PyTorch on the device
        _, _, rinv = fp8.quantize_with(x.cpu(), cpu_state, e5m2=e5m2, transpose=transpose)
        assert torch.allclose(inv.cpu(), rinv, rtol=1e-6), k
        fmax = fp8.E5M2_MAX if e5m2 else fp8.E4M3_MAX
        amax_used = x.float().abs().max() if used is None else used
        ref = (x.float() * (torch.full_like(amax_used, fmax) / amax_used)).clamp(-fmax, fmax).to(q.dtype)       # true division, as in the kernel
        assert torch.equal(q.view(torch.uint8), ref.view(torch.uint8)), k
        if transpose:
            assert qt.is_contiguous() and torch.equal(qt.view(torch.uint8), ref.t().contiguous().view(torch.uint8)), k
        assert torch.allclose(dev_state.amax3.cpu(), cpu_state.amax3), k
    # current scaling through the transposing kernel
    x = torch.randn(*shape, device="cuda").to(torch.bfloat16)
    q, qt, inv = fp8.quantize_with(x, None, e5m2=e5m2, transpose=transpose)
    q2, inv2 = fp8.quantize(x, e5m2)
    assert torch.equal(q.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(inv, inv2)
    if transpose:
        assert torch.equal(qt.view(torch.uint8), q2.t().contiguous().view(torch.uint8))


def test_gemm_fp8_mixes_formats_and_takes_two_scales():
    torch.manual_seed(4)
    a = torch.randn(256, 512, device="cuda").to(torch.float8_e5m2)
    b = torch.randn(384, 512, device="cuda").to(torch.float8_e4m3fn)
    s1, s2 = torch.tensor([0.5], device="cuda"), torch.tensor([0.25], device="cuda")
    got = torch.ops.sjb200.gemm_fp8(a, b, s1, True, 0, s2)
    ref = (a.float() @ b.float().t()) * 0.125
    assert torch.allclose(got, ref, rtol=1e-4, atol=1e-2)
    got = torch.ops.sjb200.gemm_fp8(b, a, s1, True, 0, None)
    assert torch.allclose(got, (b.float() @ a.float().t()) * 0.5, rtol=1e-4, atol=1e-2)
    # bias added in the epilogue, also when the contraction is split (only the first split adds it)
    bias = torch.randn(384, device="cuda")
    for split in (0, 1, 4):
        got = torch.ops.sjb200.gemm_fp8(a, b, s1, True, split, s2, bias)
        assert torch.allclose(got, ref + bias, rtol=1e-4, atol=1e-2), split
    got16 = torch.ops.sjb200.gemm_fp8(a, b, s1, False, 0, s2, bias)
    assert got16.dtype == torch.bfloat16 and torch.allclose(got16.float(), ref + bias, rtol=2e-2, atol=0.5)


def test_fp8_linear_returns_the_autocast_dtype():
    x = torch.randn(64, 128, device="cuda")
    w = torch.randn(256, 128, device="cuda", requires_grad=True)
    b = torch.randn(256, device="cuda", requires_grad=True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = fp8.linear(x, w, b)
        with torch.no_grad():
            y2 = fp8.linear(x, w, b, fp8.LinearScaling())
    assert y.dtype == torch.bfloat16 and y2.dtype == torch.bfloat16
    assert fp8.linear(x, w, b).dtype == torch.float32
    ref = torch.nn.functional.linear(x, w, b)
    assert torch.nn.functional.cosine_similarity(y.float().flatten(), ref.flatten(), dim=0) > 0.995
    y.float().sum().backward()
    assert torch.allclose(b.grad, torch.full_like(b, 64.0))


@pytest.mark.parametrize("delayed", [False, True])
def test_fp8_linear_all_three_products_close_to_fp32(delayed):
    torch.manual_seed(5)
    x = (torch.rand(4, 256, 512, device="cuda") < 0.25).to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(768, 512, device="cuda") * 0.03).requires_grad_(True)
    sc = fp8.LinearScaling() if delayed else None
    g = torch.randn(4, 256, 768, device="cuda", dtype=torch.bfloat16)
    from spikingjelly_b200.ops import counters
    for _ in range(3):
        x.grad = w.grad = None
        before = counters.by_name().get("gemm_fp8", 0)
        fp8.linear(x, w, None, sc).backward(g)
    assert counters.by_name().get("gemm_fp8", 0) - before == 3          # forward, data gradient, weight gradient
    xr, wr = x.detach().float().requires_grad_(True), w.detach().clone().requires_grad_(True)
    torch.nn.functional.linear(xr, wr).backward(g.float())
    cos = lambda a, b_: torch.nn.functional.cosine_similarity(a.flatten().float(), b_.flatten().float(), dim=0).item()
    assert cos(x.grad, xr.grad) > 0.99 and cos(w.grad, wr.grad) > 0.99, (cos(x.grad, xr.grad), cos(w.grad, wr.grad))
