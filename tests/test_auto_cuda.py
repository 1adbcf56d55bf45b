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
