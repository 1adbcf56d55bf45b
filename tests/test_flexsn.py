"""FlexSN: torch/hop paths, tracing + code generation + nvcc build (CPU), compiled kernels vs eager scan (GPU)."""
import copy
import functools

import pytest
import torch
import torch.nn as nn

from spikingjelly_b200.activation_based import functional, neuron, surrogate
from spikingjelly_b200.activation_based.neuron.flexsn import FlexSN, _core_requires_grad, eager_scan
from spikingjelly_b200.ops import flexsn as K

_sg = surrogate.Sigmoid()


def lif_core(x, v):
    h = v + (x - v) / 2.0
    s = _sg(h - 1.0)
    return s, h * (1.0 - s)


def cuba_core(x, gate, i, v):
    """Two inputs, two states, two outputs: current-based LIF with a multiplicative gate."""
    i = i * 0.8 + x * torch.sigmoid(gate)
    h = v + (i - v) / 4.0
    s = surrogate.ATan.spiking_function(h - 0.5, 2.0)
    return s, h, i, torch.where(s > 0, torch.zeros_like(h), h)


def test_torch_backend_matches_lif_node():
    x = torch.rand(6, 3, 5) * 2
    m = FlexSN(lif_core, 1, 1, 1, backend="torch")
    ref = neuron.LIFNode(tau=2.0, surrogate_function=surrogate.Sigmoid(), step_mode="m")
    assert torch.equal(m(x), ref(x))
    assert torch.allclose(m.states[0], ref.v)
    functional.reset_net(m)
    assert m.states is None
    m.store_state_seqs = True
    m(x)
    assert m.state_seqs[0].shape == x.shape and torch.equal(m.state_seqs[0][-1], m.states[0])


def test_single_step_and_hop_backends():
    x = torch.rand(4, 7) * 2
    ms = FlexSN(lif_core, 1, 1, 1, step_mode="s", backend="torch")
    mh = FlexSN(lif_core, 1, 1, 1, backend="hop")
    mt = FlexSN(lif_core, 1, 1, 1, backend="torch")
    assert torch.equal(mh(x), mt(x))
    ys = []
    for t in range(4):
        ys.append(ms(x[t]))
    assert torch.equal(torch.stack(ys), mt.__class__(lif_core, 1, 1, 1, backend="torch")(x))
    with pytest.raises(RuntimeError):
        ms.backend = "triton"
    with pytest.raises(ValueError):
        FlexSN(lif_core, 0, 1, 1, step_mode="m", backend="torch")


def test_empty_sequence_needs_templates_on_torch_backend():
    calls = []

    def core(x, v):
        calls.append(1)
        return x + v, v

    m = FlexSN(core, 1, 1, 1, backend="torch")
    with pytest.raises(ValueError):
        m(torch.zeros(0, 3))
    m = FlexSN(core, 1, 1, 1, backend="torch", example_outputs=(torch.zeros(3),))
    y = m(torch.zeros(0, 3))
    assert y.shape == (0, 3) and not calls and m.states[0].shape == (3,)


def test_core_requires_grad_detection():
    w = torch.ones(3, requires_grad=True)

    class Functor:
        def __init__(self):
            self.w = w

        def __call__(self, x, v):
            return x * self.w, v

        def method(self, x, v):
            return x * self.w, v

    assert _core_requires_grad(Functor()) and _core_requires_grad(Functor().method)
    assert _core_requires_grad(functools.partial(lambda x, v, k: (x * k, v), k=w))
    assert _core_requires_grad(nn.Linear(2, 2)) and not _core_requires_grad(lif_core)


def test_trace_codegen_and_build_without_gpu():
    g = K.trace_step(cuba_core, 2, 2, 2)
    assert g.joint is not None and len(g.signature) == 64
    src = K.emit_module(g)
    assert "step_fwd" in src and "step_bwd" in src and "atanf" not in src.split("step_bwd")[0].split("step_fwd")[1][:0]
    if K.nvcc_path() is None:
        pytest.skip("nvcc not present")
    so = K.compile_module(src, "cuba", load=False)
    assert so.exists() and K.compile_module(src, "cuba", load=False) == so       # second call is a cache hit
    m = FlexSN(cuba_core, 2, 2, 2, backend="triton")
    assert m.kernel_available
    # CPU tensors run the eager scan whatever the backend
    x, gate = torch.rand(5, 8), torch.randn(5, 8)
    s, h = m(x, gate)
    ref = eager_scan(cuba_core, 2, 2, 2, False, x, gate, torch.zeros(8), torch.zeros(8))
    assert torch.equal(s, ref[0]) and torch.equal(h, ref[1])
    m2 = copy.deepcopy(m)
    assert m2.kernel_available and m2._handle != m._handle


def test_unsupported_core_falls_back():
    table = torch.arange(8.0)

    def captured(x, v):
        return x + table, v

    def matmul(x, v):
        return x @ x.t(), v

    for core in (captured, matmul):
        with pytest.raises(K.UnsupportedCore):
            K.trace_step(core, 1, 1, 1, example_inputs=(torch.zeros(8, 8), torch.zeros(8, 8)) if core is matmul else None)
    m = FlexSN(captured, 1, 1, 1, backend="triton")
    assert not m.kernel_available and "UnsupportedCore" in m._build_error
    assert m(torch.zeros(2, 8)).shape == (2, 8)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("n", [4096, 1001])
def test_kernel_matches_eager_scan(dtype, n):
    dev = "cuda"
    torch.manual_seed(0)
    T = 6
    x = (torch.rand(T, n, device=dev) * 2).to(dtype)
    gate = torch.randn(T, n, device=dev).to(dtype)
    i0 = (torch.rand(n, device=dev) * 0.2).to(dtype)
    v0 = (torch.rand(n, device=dev) * 0.2).to(dtype)
    m = FlexSN(cuba_core, 2, 2, 2, backend="triton", store_state_seqs=True)
    assert m.kernel_available
    leaves = [t.clone().requires_grad_(True) for t in (x, gate, i0, v0)]
    m.states = [leaves[2], leaves[3]]
    s, h = m(leaves[0], leaves[1])
    w1, w2 = torch.randn_like(s), torch.randn_like(h)
    loss = (s * w1).sum() + (h * w2).sum() + m.state_seqs[0].sum() * 0.1 + (m.states[1] * 0.3).sum()
    loss.backward()

    ref_leaves = [t.clone().float().requires_grad_(True) for t in (x, gate, i0, v0)]
    r = eager_scan(cuba_core, 2, 2, 2, True, *ref_leaves)
    (r[0] * w1.float()).sum().add((r[1] * w2.float()).sum()).add(r[2].sum() * 0.1).add((r[3][-1] * 0.3).sum()).backward()
    if dtype == torch.float32:
        assert torch.equal(s, r[0]) and torch.allclose(h, r[1], atol=1e-6)
        for a, b in zip(leaves, ref_leaves):
            assert torch.allclose(a.grad, b.grad, atol=1e-5, rtol=1e-5)
    else:
        # the kernel keeps fp32 between operators; compare against the fp32 scan of the same rounded inputs
        flip = (s.float() != r[0]).float().mean().item()
        assert flip < 0.02
        tol = 0.05 if dtype == torch.float16 else 0.2
        for a, b in zip(leaves, ref_leaves):
            err = (a.grad.float() - b.grad).abs().mean() / (b.grad.abs().mean() + 1e-6)
            assert err < tol + 4 * flip


@pytest.mark.gpu
def test_kernel_lif_equals_builtin_lif_and_counts_launches():
    from spikingjelly_b200.ops import counters
    x = torch.rand(4, 8, 512, device="cuda") * 2
    m = FlexSN(lif_core, 1, 1, 1, backend="triton")
    ref = neuron.LIFNode(tau=2.0, surrogate_function=surrogate.Sigmoid(), step_mode="m", backend="cuda")
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    before = counters.by_name().get("flexsn_forward", 0)
    ya, yb = m(xa), ref(xb)
    assert counters.by_name().get("flexsn_forward", 0) == before + 1
    assert torch.equal(ya, yb)
    g = torch.randn_like(ya)
    ya.backward(g)
    yb.backward(g)
    assert torch.allclose(xa.grad, xb.grad, atol=1e-6, rtol=1e-5)
    with torch.no_grad():
        functional.reset_net(m)
        assert torch.equal(m(x), yb.detach())
        outs = m.kernel(x, torch.zeros_like(x[0]))
        assert torch.equal(outs[0], yb.detach()) and torch.equal(outs[1][-1], m.states[0])


@pytest.mark.gpu
def test_library_neurons_without_handwritten_kernels_run_compiled():
    """Izhikevich, integer LIF and the ternary IF neuron: compiled multi-step path == eager path."""
    from spikingjelly_b200.ops import counters
    torch.manual_seed(0)
    x = torch.rand(6, 4, 256, device="cuda") * 2
    before = counters.by_name().get("flexsn_forward", 0)
    for make in (lambda b: neuron.IzhikevichNode(step_mode="m", backend=b, a=0.2, b=0.05),
                 lambda b: neuron.ILIFNode(step_mode="m", backend=b)):
        a, e = make("cuda"), make("torch")
        xa, xe = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
        ya, ye = a(xa), e(xe)
        assert torch.equal(ya, ye), type(a).__name__
        g = torch.randn_like(ya)
        ya.backward(g)
        ye.backward(g)
        assert torch.allclose(xa.grad, xe.grad, atol=1e-5, rtol=1e-4), type(a).__name__
        assert torch.allclose(a.v, e.v, atol=1e-6)
    st = neuron.STBIFNeuron(0.25, level=8, step_mode="m").cuda()
    ref = neuron.STBIFNeuron(0.25, level=8, step_mode="m")
    xs = torch.randn(5, 3, 64, device="cuda")
    with torch.no_grad():
        out = st(xs)
        want = ref(xs.cpu())
    assert torch.allclose(out.cpu(), want) and torch.allclose(st.acc_q.cpu(), ref.acc_q)
    assert counters.by_name().get("flexsn_forward", 0) >= before + 3
    with torch.inference_mode():                     # buffers created here have no version counter
        st2 = neuron.STBIFNeuron(0.25, level=8, step_mode="m").cuda()
        assert torch.allclose(st2(xs).cpu(), want)
