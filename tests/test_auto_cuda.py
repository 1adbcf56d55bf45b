"""Hand-assembled kernels of ``cuda_kernel/auto_cuda/base.py``: source assembly and argument checks on the CPU, launches
on the GPU (element-wise, sequence forward and reverse, half2 with odd sizes)."""
import pytest
import torch

from spikingjelly_b200.activation_based.cuda_kernel.auto_cuda import base


def _axpy():
    k = base.CKernel1D("sjb200_test_axpy")
    k.add_param("const float *", "x")
    k.add_param("float *", "y")
    k.add_param("const float &", "a")
    k.core = "        y[index] = a * x[index] + y[index];"
    return k


def test_source_assembly_and_checks():
    k = _axpy()
    src = k.full_codes
    assert 'extern "C" __global__' in src and "void sjb200_test_axpy(const int numel, const float * x, float * y, const float a)" in src
    assert "if (index < numel)" in src and "//------core start------" in src and "launch_sjb200_test_axpy" in k.translation_unit
    with pytest.raises(ValueError):
        k.add_param("float *", "x")
    with pytest.raises(ValueError):
        k.add_param("int", "index")
    assert k.check_attributes(kernel_name="sjb200_test_axpy") and not k.check_attributes(kernel_name="other")
    with pytest.raises(ValueError, match="missing"):
        k.check_keys({"x": 1})
    with pytest.raises(TypeError):
        k.check_ctypes({"numel": 4, "x": torch.zeros(4, dtype=torch.float64), "y": torch.zeros(4), "a": 1.0})
    with pytest.raises(TypeError):
        k.check_ctypes({"numel": 4, "x": torch.zeros(4), "y": torch.zeros(4), "a": torch.zeros(1)})
    k2 = base.CKernel2D("seq", reverse=True)
    k2.pre_core, k2.post_core = "float v = 0.0f;", "v_last[index] = v;"
    assert "for (int t = numel - N + index; t >= 0; t -= dt)" in k2.full_codes and "pre_core start" in k2.full_codes and "post_core start" in k2.full_codes
    with pytest.raises(ValueError):
        k2.check_shape({"a": torch.zeros(3, 4), "b": torch.zeros(3, 5)})
    typer = base.CodeTyper(4)
    typer.append("a = b; c = d")
    with base.CodeBlock(typer):
        typer.append("e = f;")
    assert typer.codes == "\n    a = b;\n    c = d;\n    {\n     e = f;\n    }\n"
    assert base.wrap_with_comment("", "x") == "" and base.startswiths("half2 *", ("half", "float"))


def test_translation_unit_compiles_for_sm100a():
    from spikingjelly_b200.ops.flexsn import compiler
    if compiler.nvcc_path() is None:
        pytest.skip("nvcc not available")
    assert str(compiler.compile_module(_axpy().translation_unit, name="auto_cuda_sjb200_test_axpy", load=False)).endswith(".so")


@pytest.mark.gpu
def test_elementwise_launch():
    x = torch.randn(1000, device="cuda")
    y = torch.randn(1000, device="cuda")
    want = 2.5 * x + y
    out = _axpy().simple_call(x=x, y=y, a=2.5)
    assert torch.allclose(out["y"], want)


@pytest.mark.gpu
@pytest.mark.parametrize("reverse", [False, True])
def test_sequence_kernel(reverse):
    k = base.CKernel2D("sjb200_test_scan_r" if reverse else "sjb200_test_scan", reverse=reverse)
    k.add_param("const float *", "x_seq")
    k.add_param("float *", "v_seq")
    k.add_param("float *", "v_last")
    k.add_param("const float &", "decay")
    k.pre_core = "        float v = 0.0f;"
    k.core = "            v = v * decay + x_seq[t];\n            v_seq[t] = v;"
    k.post_core = "        v_last[index] = v;"
    x = torch.randn(7, 333, device="cuda")
    out = k.simple_call(x_seq=x, v_seq=torch.empty_like(x), v_last=torch.empty(333, device="cuda"), decay=0.5)
    v, want = torch.zeros(333, device="cuda"), torch.empty_like(x)
    for t in (range(6, -1, -1) if reverse else range(7)):
        v = v * 0.5 + x[t]
        want[t] = v
    assert torch.allclose(out["v_seq"], want, atol=1e-6) and torch.allclose(out["v_last"], v, atol=1e-6)


@pytest.mark.gpu
def test_half2_kernel_pads_odd_sizes():
    k = base.CKernel1D("sjb200_test_h2")
    k.add_param("const half2 *", "x")
    k.add_param("half2 *", "y")
    k.core = "        y[index] = __hadd2(x[index], x[index]);"
    x = torch.randn(1001, device="cuda", dtype=torch.float16)
    out = k.simple_call(x=x, y=torch.empty_like(x))
    assert out["y"].shape == x.shape and torch.equal(out["y"], x + x)


def _lif_charge(x: torch.Tensor, v_last: torch.Tensor, v_reset: float, tau: float):
    return v_last + (x - (v_last - v_reset)) / tau


def _plif_like(x: torch.Tensor, v_last: torch.Tensor, w: torch.Tensor):
    return v_last * w + x * (1.0 - w)


def test_generator_traces_and_emits_kernels():
    from spikingjelly_b200.activation_based import surrogate
    from spikingjelly_b200.activation_based.cuda_kernel.auto_cuda import generator as G
    inputs, inter, outputs, cmds = G.analyse_graph(_lif_charge, (True, True, False, False))
    assert [n.kind for n in inputs.values()] == ["seq", "state", "scalar", "scalar"] and len(outputs) == 1
    assert [c[1] for c in cmds] == ["-", "-", "/", "+"]
    fwd, name, cuda_cmds = G.gen_forward_codes(inputs, inter, outputs, cmds, hard_reset=True)
    assert name.startswith("auto_neuron_fwd_hard_") and len(cuda_cmds) == 4
    assert "x_seq[t]" in fwd.full_codes and "spike_seq[t] = spike;" in fwd.full_codes and "v_reset" in fwd.cparams
    bwd, bname, tensors = G.gen_backward_codes(cuda_cmds, inputs, outputs, cmds, True, False, surrogate.ATan())
    assert bwd.reverse and tensors == [] and "grad_x_seq[t]" in bwd.full_codes and "surrogate_grad<1>" in bwd.full_codes
    assert G.hash_str("a") == G.hash_str("a") and len(G.hash_str("a")) == 16
    with pytest.raises(NotImplementedError):
        G.analyse_graph(lambda x, v_last: torch.exp(x) + v_last, (True, True))
    from spikingjelly_b200.ops.flexsn import compiler
    if compiler.nvcc_path() is not None:
        for k in (fwd, bwd):
            compiler.compile_module(k.translation_unit, name="auto_cuda_" + k.kernel_name, load=False)


@pytest.mark.gpu
@pytest.mark.parametrize("hard_reset", [True, False])
@pytest.mark.parametrize("fun,extra", [(_lif_charge, "scalars"), (_plif_like, "tensor")])
def test_generated_kernels_match_autograd(hard_reset, fun, extra):
    from spikingjelly_b200.activation_based import surrogate
    from spikingjelly_b200.activation_based.cuda_kernel.auto_cuda import generator as G
    torch.manual_seed(0)
    T, N, v_th, v_reset = 6, 500, 1.0, 0.0
    sg = surrogate.ATan()
    x = torch.randn(T, N, device="cuda") * 1.5
    v0 = torch.rand(N, device="cuda") * 0.5
    if extra == "scalars":
        w = None
        flags, kw, call = (True, True, False, False), {"v_reset": v_reset, "tau": 2.0}, lambda xt, v, w_: fun(xt, v, v_reset, 2.0)
    else:
        w = torch.rand(N, device="cuda") * 0.5 + 0.25
        flags, kw, call = (True, True, True), {"w": w}, lambda xt, v, w_: fun(xt, v, w_)
        if hard_reset:
            kw["v_reset"] = v_reset
    inputs, inter, outputs, cmds = G.analyse_graph(fun, flags)
    fwd, _, cuda_cmds = G.gen_forward_codes(inputs, inter, outputs, cmds, hard_reset)
    bwd, _, tensors = G.gen_backward_codes(cuda_cmds, inputs, outputs, cmds, hard_reset, False, sg)
    fkw = bkw = kw                      # the charge rule's own v_reset argument doubles as the reset value
    reset_kw = {}
    out = fwd.simple_call(x_seq=x, v_init=v0, spike_seq=torch.empty_like(x), h_seq=torch.empty_like(x), v_v_seq=torch.empty_like(x), v_th=v_th,
                          **fkw)
    # autograd oracle
    xr, vr = x.clone().requires_grad_(True), v0.clone().requires_grad_(True)
    wr = w.clone().requires_grad_(True) if w is not None else None
    v, spikes, vs = vr, [], []
    for t in range(T):
        h = call(xr[t], v, wr)
        s = sg(h - v_th)
        v = s * v_reset + (1 - s) * h if hard_reset else h - s * v_th
        spikes.append(s)
        vs.append(v)
    S, V = torch.stack(spikes), torch.stack(vs)
    assert torch.equal(out["spike_seq"], S.detach()) and torch.allclose(out["v_v_seq"], V.detach(), atol=1e-6)
    gs, gv = torch.randn_like(S), torch.randn_like(V) * 0.1
    wanted = [xr, vr] + ([wr] if wr is not None else [])
    grads = torch.autograd.grad([S, V], wanted, [gs, gv])
    extra_out = {f"grad_{n}": torch.empty(N, device="cuda") for n in tensors}
    res = bwd.simple_call(grad_spike_seq=gs, grad_v_seq=gv, h_seq=out["h_seq"], v_v_seq=out["v_v_seq"], v_init=v0, x_seq=x,
                          grad_x_seq=torch.empty_like(x), grad_v_init=torch.empty(N, device="cuda"), v_th=v_th, **bkw, **reset_kw, **extra_out)
    assert torch.allclose(res["grad_x_seq"], grads[0], rtol=1e-4, atol=1e-5)
    assert torch.allclose(res["grad_v_init"], grads[1], rtol=1e-4, atol=1e-5)
    if wr is not None:
        assert torch.allclose(res["grad_w"], grads[2], rtol=1e-4, atol=1e-4)
