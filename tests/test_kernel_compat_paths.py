"""``activation_based.cuda_kernel`` / ``triton_kernel`` import paths: spike storage, memory-saving spike layers, helpers."""
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from spikingjelly_b200 import configure
from spikingjelly_b200.activation_based.cuda_kernel import cuda_utils, spike_op, tensor_cache
from spikingjelly_b200.activation_based.triton_kernel import bit_spike_compress, bit_spike_decompress, fp8_capability


def test_spike_bit_round_trip_and_cache():
    torch.manual_seed(0)
    s = (torch.rand(3, 5, 7) < 0.4).float()
    packed, dt, shape, pad = tensor_cache.float_spike_to_bool(s)
    assert packed.dtype == torch.uint8 and packed.numel() == (s.numel() + 7) // 8 and pad == (8 - s.numel() % 8) % 8
    assert torch.equal(tensor_cache.bool_spike_to_float(packed, dt, shape, pad), s)
    assert torch.equal(bit_spike_decompress(bit_spike_compress(s), s.shape, torch.float32), s)
    for level in (0, 1):
        old = configure.save_bool_spike_level
        configure.save_bool_spike_level = level
        try:
            cache = tensor_cache.BoolTensorCache()
            k1, k2 = cache.store_bool(s), cache.store_bool(s)
            assert k1 == k2 and len(cache.cache) == 1
            assert torch.equal(cache.get_float(k1, s.shape), s) and len(cache.cache) == 1
            assert torch.equal(cache.get_float(k2, s.shape), s) and len(cache.cache) == 0
        finally:
            configure.save_bool_spike_level = old


def test_helpers():
    assert cuda_utils.cal_blocks(1000, 256) == 4 and cuda_utils.cal_blocks(1024) == 1024 // configure.cuda_threads
    assert cuda_utils.cpu_timer(lambda: sum(range(100))) >= 0
    assert cuda_utils.cal_fun_t(3, "cpu", lambda: None) >= 0
    a, = cuda_utils.get_contiguous(torch.arange(6).view(2, 3).t())
    assert a.is_contiguous()
    cap = fp8_capability.fp8_capability()
    assert "available" in cap and fp8_capability.is_fp8_dtype(torch.float8_e4m3fn) and not fp8_capability.is_fp8_dtype(torch.float16)
    lin = spike_op.SpikeLinear(4, 3)
    x = (torch.rand(2, 4) < 0.5).float()
    torch.testing.assert_close(lin(x), F.linear(x, lin.weight, lin.bias))        # CPU: the plain operator


@pytest.mark.gpu
@pytest.mark.parametrize("level", [0, 1])
def test_spike_layers_match_plain_layers_on_gpu(level):
    old = configure.save_bool_spike_level
    configure.save_bool_spike_level = level
    try:
        torch.manual_seed(0)
        for spike_mod, plain, shape in ((spike_op.SpikeLinear(16, 8), nn.Linear(16, 8), (4, 16)),
                                        (spike_op.SpikeConv1d(4, 6, 3, padding=1), nn.Conv1d(4, 6, 3, padding=1), (2, 4, 10)),
                                        (spike_op.SpikeConv2d(4, 6, 3, stride=2, padding=1), nn.Conv2d(4, 6, 3, stride=2, padding=1), (2, 4, 9, 9)),
                                        (spike_op.SpikeConv3d(2, 3, 3, padding=1), nn.Conv3d(2, 3, 3, padding=1), (2, 2, 5, 5, 5))):
            spike_mod, plain = spike_mod.cuda(), plain.cuda()
            plain.load_state_dict(spike_mod.state_dict())
            x = (torch.rand(*shape, device="cuda") < 0.3).float().requires_grad_(True)
            xr = x.detach().clone().requires_grad_(True)
            y, yr = spike_mod(x), plain(xr)
            torch.testing.assert_close(y, yr)
            g = torch.randn_like(y)
            y.backward(g); yr.backward(g)
            torch.testing.assert_close(x.grad, xr.grad)
            torch.testing.assert_close(spike_mod.weight.grad, plain.weight.grad)
            torch.testing.assert_close(spike_mod.bias.grad, plain.bias.grad)
        assert len(tensor_cache.BOOL_TENSOR_CACHE.cache) == 0
    finally:
        configure.save_bool_spike_level = old


def test_cfunction_expression_builders():
    import math
    from spikingjelly_b200.activation_based.cuda_kernel.auto_cuda import cfunction as cf
    assert cf.mul(None, "a", "b", "float") == "(a * b)" and cf.mul("z", "a", "1.0f", "float") == "z = a;"
    assert cf.add("z", "0.0f", "b", "float") == "z = b;" and cf.sub(None, "a", "b", "half2") == "(__hsub2(a, b))"
    assert cf.mul(None, "__float2half2_rn(1.0f)", "b", "half2") == "(b)"
    assert cf.heaviside("s", "h - v_th", "float") == "s = (float) (h - v_th >= 0.0f);"
    assert cf.constant(None, 2, "float") == "(2.0f)" and "__float2half2_rn" in cf.constant("c", 0.5, "half2")
    nested = cf.if_else_else("w", "x", "y", "z", "mx", "my", "float")
    assert nested.startswith("w = x * mx + (y * my + z * (1.0f - my)) * (1.0f - mx)")
    with pytest.raises(NotImplementedError):
        cf.add(None, "a", "b", "double")
    # the fp32 surrogate formulas are plain C: evaluate them with Python after translating the math calls
    def evaluate(code, v):
        expr = code.split("=", 1)[1].rstrip(";")
        for c_name, py in (("expf", "math.exp"), ("fabsf", "abs"), ("__powf", "pow"), ("fminf", "min")):
            expr = expr.replace(c_name, py)
        import re
        expr = re.sub(r"(\d)f\b", r"\1", expr)
        expr = re.sub(r"\(([^()?]+)\?([^:()]+):([^()]+)\)", r"((\2) if (\1) else (\3))", expr)
        return eval(expr, {"math": math, "abs": abs, "pow": pow, "min": min, "x": v})
    from spikingjelly_b200.activation_based import surrogate
    for v in (-0.7, 0.0, 0.3):
        xt = torch.tensor(v, dtype=torch.float64, requires_grad=True)
        surrogate.Sigmoid(alpha=4.0)(xt).backward()
        assert evaluate(cf.sigmoid_backward("g", "x", 4.0, "float"), v) == pytest.approx(float(xt.grad), rel=1e-6)
        xt = torch.tensor(v, dtype=torch.float64, requires_grad=True)
        surrogate.ATan(alpha=2.0)(xt).backward()
        assert evaluate(cf.atan_backward("g", "x", 2.0, "float"), v) == pytest.approx(float(xt.grad), rel=1e-6)
    assert "__floats2half2_rn(g_lo, g_hi)" in cf.sigmoid_backward("g", "x", 4.0, "half2")


def test_triton_utils_names_and_execution_plan():
    import torch
    from spikingjelly_b200.activation_based.triton_kernel import triton_utils as U
    from spikingjelly_b200.activation_based.triton_kernel.neuron_kernel import utils as plan_mod
    assert U.normalize_triton_compute_dtype_name("torch.float16") == "fp16" and U.normalize_triton_compute_dtype_name(torch.bfloat16) == "bf16"
    assert U.normalize_triton_storage_dtype("e5m2") is torch.float8_e5m2 and U.normalize_triton_storage_dtype(torch.float16) is torch.float16
    assert U.is_fp8_dtype(torch.float8_e4m3fn) and not U.is_fp8_dtype(torch.float16)
    assert U.triton_neuron_dtype_id_to_torch_dtype(U.torch_dtype_to_triton_neuron_dtype_id(torch.bfloat16)) is torch.bfloat16
    assert U.triton_compute_dtype_name_to_neuron_dtype_id("fp8", torch.float8_e4m3fn) == U.TRITON_NEURON_DTYPE_FP8_E4M3FN
    assert U.torch_dtype_for_triton_compute_dtype("fp8", torch.float8_e5m2) is torch.float8_e5m2
    assert U.use_static_range_for_triton_neuron_kernel(4) and not U.use_static_range_for_triton_neuron_kernel(16)
    import pytest
    for bad in (lambda: U.normalize_triton_compute_dtype_name("int8"), lambda: U.normalize_triton_storage_dtype("int8"),
                lambda: U.triton_compute_dtype_name_to_neuron_dtype_id("fp8", torch.float16), lambda: U.normalize_cuda_device("cpu")):
        with pytest.raises(ValueError):
            bad()
    plan = plan_mod.prepare_triton_neuron_execution_plan(neuron_type="lif", device="cuda:0", storage_dtype="fp8_e4m3fn", spike_dtype=torch.bfloat16)
    assert plan.storage_dtype is torch.float8_e4m3fn and plan.forward_compute_dtype_name == "fp32" and plan.spike_dtype_id == 2
    assert plan.matches(neuron_type="lif", device=0, storage_dtype=torch.float8_e4m3fn, forward_compute_dtype="float32", spike_dtype=torch.bfloat16,
                        save_intermediates=True)
    assert not plan.matches(neuron_type="if", device=0, storage_dtype=torch.float8_e4m3fn, forward_compute_dtype="fp32", spike_dtype=torch.bfloat16,
                            save_intermediates=True)
    with pytest.raises(ValueError):
        plan_mod.prepare_triton_neuron_execution_plan(neuron_type="qif", device=0, storage_dtype="fp32")
    with pytest.raises(ValueError):
        plan_mod.prepare_triton_neuron_execution_plan(neuron_type="lif", device=0, storage_dtype="fp16", forward_compute_dtype="fp8")

    @U.contiguous_and_device_guard
    def probe(a, b=None):
        return a.is_contiguous() and (b is None or b.is_contiguous())
    assert probe(torch.arange(6).view(2, 3).t(), b=torch.arange(6).view(2, 3).t())


@pytest.mark.gpu
def test_functional_neuron_kernels_match_the_modules():
    import torch
    from spikingjelly_b200.activation_based import neuron, surrogate
    from spikingjelly_b200.activation_based.triton_kernel.neuron_kernel import lif as K
    torch.manual_seed(0)
    sg = surrogate.ATan()
    x = torch.randn(6, 4, 64, device="cuda", requires_grad=True)
    s, v_seq = K.multistep_lif(x, torch.zeros(4, 64, device="cuda"), True, 2.0, 1.0, 0.0, False, sg)
    node = neuron.LIFNode(tau=2.0, surrogate_function=sg, step_mode="m", backend="cuda", store_v_seq=True).cuda()
    x2 = x.detach().clone().requires_grad_(True)
    s2 = node(x2)
    assert torch.equal(s, s2) and torch.equal(v_seq, node.v_seq)
    g = torch.randn_like(s)
    s.backward(g)
    s2.backward(g)
    assert torch.equal(x.grad, x2.grad)
    xb = torch.randn(6, 4, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    s8, v8, h8 = K.multistep_lif_mp(xb, torch.zeros(4, 64, device="cuda"), decay_input=True, tau=2.0, v_threshold=1.0, v_reset=0.0,
                                    storage_dtype="fp8_e4m3fn", spike_dtype=torch.bfloat16, surrogate_function=sg)
    assert s8.dtype == torch.bfloat16 and h8 is None and v8.shape == xb.shape
    g8 = torch.randn_like(s8)
    s8.backward(g8)
    assert xb.grad is not None and xb.grad.dtype == torch.bfloat16
    # same spikes AND the same gradient as the bf16 kernel fed with the e4m3-rounded input: the cast to the storage type
    # happens inside the autograd function, so the gradient is not rounded to fp8 on its way back
    xw = xb.detach().to(torch.float8_e4m3fn).to(torch.bfloat16).requires_grad_(True)
    ref, _ = K.multistep_lif(xw, torch.zeros(4, 64, device="cuda", dtype=torch.bfloat16), True, 2.0, 1.0, 0.0, False, sg)
    ref.backward(g8)
    assert torch.equal(s8, ref) and torch.equal(xb.grad, xw.grad)
    # a prepared plan gives the same result as the keyword form; PLIF takes the reciprocal time constant as a tensor
    from spikingjelly_b200.activation_based.triton_kernel.neuron_kernel import integrate_and_fire as KI, plif as KP, utils as KU
    plan = KU.prepare_triton_neuron_execution_plan(neuron_type="lif", device=xb.device, storage_dtype="fp8_e4m3fn", spike_dtype=torch.bfloat16)
    s9, _, _ = K.multistep_lif_mp_with_plan(xb.detach(), torch.zeros(4, 64, device="cuda"), plan, decay_input=True, tau=2.0, v_threshold=1.0,
                                            v_reset=0.0, surrogate_function=sg)
    assert torch.equal(s9, s8)
    with pytest.raises(ValueError):
        KI.multistep_if_mp_with_plan(xb.detach(), torch.zeros(4, 64, device="cuda"), plan, v_threshold=1.0, v_reset=0.0)
    r_tau = torch.tensor(0.5, device="cuda", requires_grad=True)
    xp = x.detach().clone().requires_grad_(True)
    sp, vp, _ = KP.multistep_plif_mp(xp, torch.zeros(4, 64, device="cuda"), r_tau, decay_input=True, v_threshold=1.0, v_reset=0.0,
                                     storage_dtype="fp32", surrogate_function=sg)
    assert torch.equal(sp, s2.detach())                       # 1 / tau = 0.5 is the LIF above
    sp.backward(g)
    assert r_tau.grad is not None and torch.allclose(xp.grad, x2.grad)
    si, vi = K.multistep_lif_inference(x.detach(), torch.zeros(4, 64, device="cuda"), True, 2.0, 1.0, 0.0, False, True)
    assert torch.equal(si, s2.detach()) and torch.equal(vi, node.v_seq) and not si.requires_grad


def test_object_handles_switch_and_raw_arguments(monkeypatch):
    import ctypes
    import gc
    import numpy as np
    import torch
    from spikingjelly_b200.activation_based.cuda_kernel import cuda_utils as U

    class Thing:
        pass
    a, b = Thing(), Thing()
    ha, hb = U.register_python_object(a), U.register_python_object(b)
    assert ha != hb and U.register_python_object(a) == ha and U.resolve_python_object(hb) is b
    del a
    gc.collect()
    with pytest.raises(RuntimeError, match="Unknown python object"):
        U.resolve_python_object(ha)
    monkeypatch.setenv("SJ_USE_CUPY_OP", "off")
    assert U.use_cupy_custom_op() is False
    with pytest.raises(TypeError):
        U.wrap_args_to_raw_kernel(0, "text")
    out = U.wrap_args_to_raw_kernel(-1, 3, 2.5, np.float32(1.0), True)
    assert [type(v) for v in out] == [ctypes.c_int, ctypes.c_float, ctypes.c_float, ctypes.c_bool] and out[1].value == 2.5
    with pytest.raises(ValueError):
        U.wrap_args_to_raw_kernel(0, torch.zeros(2))              # a CPU tensor is on device -1


def test_reference_submodule_import_paths():
    """Modules the reference splits into several files resolve here too (same names, one implementation)."""
    import importlib
    for path, names in (("activation_based.neuron.noisy", ["NoisyCUBALIFNode", "powerlaw_psd_gaussian"]),
                        ("activation_based.neuron.plif", ["ParametricLIFNode"]),
                        ("activation_based.neuron.spikezip", ["STBIFNeuron"]),
                        ("activation_based.layer.stateless_wrapper", ["Conv2d", "WSLinear"]),
                        ("activation_based.op_counter.synop", ["SynOpCounter"]),
                        ("activation_based.op_counter.neuromc.mux_counter", ["NeuroMCMuxCounter"]),
                        ("activation_based.precision.float8_te", []),
                        ("activation_based.distributed.pipeline.partition", []),
                        ("activation_based.distributed.tensor_parallel.linear", []),
                        ("activation_based.distributed.adapters.base", [])):
        m = importlib.import_module("spikingjelly_b200." + path)
        for n in names:
            assert hasattr(m, n), (path, n)
    import spikingjelly_b200.activation_based.distributed.pipeline.runtime as r
    assert r.__name__ == "spikingjelly_b200.parallel.pipeline"
