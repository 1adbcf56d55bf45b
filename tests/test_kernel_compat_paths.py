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
    # positional forms: surrogate as (id, alpha) in the reference's numbering (1 = ATan), dtypes as ids
    sf, vf, hf = K.multistep_lif_forward(x.detach(), torch.zeros(4, 64, device="cuda"), True, 2.0, 1.0, 0.0, False, False, 1, sg.alpha, True)
    assert torch.equal(sf, s2.detach()) and hf is None
    from spikingjelly_b200.activation_based.triton_kernel import triton_utils as TU
    e4, b16 = TU.torch_dtype_to_triton_neuron_dtype_id(torch.float8_e4m3fn), TU.torch_dtype_to_triton_neuron_dtype_id(torch.bfloat16)
    sm, _, _ = K.multistep_lif_mp_inference(xb.detach(), torch.zeros(4, 64, device="cuda"), True, 2.0, 1.0, 0.0, False, e4, 0, b16, False)
    assert torch.equal(sm, s8.detach())
    from spikingjelly_b200.activation_based.triton_kernel.neuron_kernel import stbif as KS
    xs = torch.randn(6, 512, device="cuda") * 0.5
    args = (torch.full((512,), 0.5, device="cuda"), torch.zeros(512, device="cuda"), torch.tensor(0.25), torch.tensor(7.0), torch.tensor(-8.0))
    og, qg, ag, cg, fg = KS.multi_step_stbif(xs, *args)
    oc, qc, ac, cc, fc = KS.multi_step_stbif(xs.cpu(), *(a.cpu() for a in args))
    assert torch.equal(og.cpu(), oc) and torch.equal(ag.cpu(), ac) and torch.equal(qg.cpu(), qc) and bool(fg) == bool(fc)
    from spikingjelly_b200.activation_based.cuda_kernel.neuron_kernel.multi_step import izhikevich as KZ, lif as KL
    sl, vl = KL.lif_multi_step(x.detach(), torch.zeros(4, 64, device="cuda"), True, 2.0, 1.0, 0.0, False, sg)
    assert torch.equal(sl, s2.detach()) and torch.equal(vl, node.v_seq)
    xz = torch.rand(5, 300, device="cuda") * 3
    z = torch.zeros(300, device="cuda")
    zg = KZ.izhikevich_multi_step(xz, z, z.clone(), 2.0, 1.0, 0.0, -0.1, 0.02, 0.2, 200.0, 0.5, 1.0, False, sg)
    zc = KZ.izhikevich_multi_step(xz.cpu(), z.cpu(), z.cpu(), 2.0, 1.0, 0.0, -0.1, 0.02, 0.2, 200.0, 0.5, 1.0, False, sg)
    assert torch.equal(zg[0].cpu(), zc[0]) and torch.allclose(zg[1].cpu(), zc[1], atol=1e-5) and torch.allclose(zg[2].cpu(), zc[2], atol=1e-5)


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


def test_compat_packages_on_cpu():
    """torch2triton, triton_kernel.flexsn, surrogate_kernel, ilif / stbif functional forms, inductor_cache: CPU behaviour."""
    import torch
    from spikingjelly_b200.activation_based import neuron, surrogate
    from spikingjelly_b200.activation_based.neuron import inductor_cache as IC
    from spikingjelly_b200.activation_based.triton_kernel import dummy, flexsn as TF, surrogate_kernel as SK, torch2triton as T2
    from spikingjelly_b200.activation_based.triton_kernel.flexsn import custom_ops as C, hop, template, wrapper
    from spikingjelly_b200.activation_based.triton_kernel.neuron_kernel import ilif, stbif
    sg = surrogate.Sigmoid(alpha=4.0)

    def core(x, v):
        h = v + (x - v) * 0.5
        s = sg(h - 1.0)
        return s, h * (1.0 - s)
    fwd, bwd = T2.generate_forward_and_backward_graph(core, (torch.rand(8), torch.rand(8)), (True, False))
    assert len([n for n in fwd.nodes if n.op == "placeholder"]) == 2 and len([n for n in bwd.nodes if n.op == "placeholder"]) == 4
    src, name = T2.generate_triton_code_str(fwd, "lif core")
    assert name.startswith("lif_core_") and f"void {name}(" in src
    fk, bk, info = TF.build_training_kernels(core, 1, 1, 1)
    assert fk is bk and info.fwd_kernel_returns == ["s0", "v0"] and info.num_fwd_kernel_returns == 2
    before = C.flexsn_kernel_registry_info()["entries"]
    h = C.register_flexsn_kernel_handle(forward_kernel=fk, backward_kernel=bk, training_info=info)
    assert C.flexsn_kernel_registry_info()["entries"] == before + 1
    C.release_flexsn_kernel_handle(h)
    assert C.flexsn_kernel_registry_info()["entries"] == before
    with pytest.raises(TypeError):
        C.register_flexsn_kernel_handle(forward_kernel=object())
    assert template.get_flexsn_backward_kernel(fk.graphs)[1] == "flexsn_backward"
    x, v0 = torch.rand(5, 8), torch.zeros(8)
    full, last = hop.eager_scan(core, 1, 1, 1, x, v0), hop.eager_scan_final_state(core, 1, 1, 1, x, v0)
    assert torch.equal(full[1][-1], last[1]) and not hop.lowerable_scan_available()
    assert [wrapper.flexsn_backward_ncl_bucket(n) for n in (1, 4097, 131073, 1048577, 8388609)] == [0, 1, 2, 3, 4]
    assert SK.resolve_sg_triton_id_and_alpha(surrogate.ATan(alpha=3.0)) == (1, 3.0)
    with pytest.raises(NotImplementedError):
        SK.resolve_sg_triton_id_and_alpha(surrogate.PiecewiseLeakyReLU())
    hh = torch.linspace(-1, 1, 7)
    assert torch.allclose(SK.sg_triton(hh, 4.0, 0), 4.0 * torch.sigmoid(4 * hh) * (1 - torch.sigmoid(4 * hh)))
    assert not dummy.DummyImport().a.b(1)[2]
    xs = torch.randn(6, 8) * 0.5
    out, q, acc, cur, flag = stbif.multi_step_stbif(xs, torch.full((8,), 0.5), torch.zeros(8), torch.tensor(0.25), torch.tensor(7.0), torch.tensor(-8.0))
    node = neuron.STBIFNeuron(0.25, level=16, sym=True, step_mode="m")
    assert torch.equal(out, node(xs)) and torch.equal(acc, node.acc_q) and bool(flag)
    xi = torch.rand(5, 4) * 3
    s, v = ilif.multistep_ilif_forward_no_grad(xi, torch.zeros(4), 0.25, 1.0, 4, True)
    ref = neuron.ILIFNode(tau=4 / 3, step_mode="m", store_v_seq=True)
    assert torch.equal(s, ref(xi)) and torch.equal(v, ref.v_seq)
    IC.clear()
    key = ("lif", IC.surrogate_key(sg), IC.runtime_key(x))
    f1 = IC.compile_graph(key, lambda: 1)
    assert IC.compile_graph(key, lambda: 2) is f1 and IC.info()["hits"] == 1 and IC.compile_graph(None, core) is core
    assert torch.equal(IC.surrogate_callable(sg)(hh), sg(hh))


@pytest.mark.gpu
def test_fragment_assembled_neuron_kernels_match_autograd():
    """IF / LIF / PLIF kernels built from code fragments (the custom-neuron extension classes) against an eager loop."""
    import torch
    from spikingjelly_b200.activation_based import functional, surrogate
    from spikingjelly_b200.activation_based.cuda_kernel.neuron_kernel.multi_step import integrate_and_fire as MI, lif as ML, plif as MP
    from spikingjelly_b200.activation_based.cuda_kernel.neuron_kernel.multi_step.base import NeuronBPTTKernel, NeuronFPTTKernel
    from spikingjelly_b200.activation_based.cuda_kernel.neuron_kernel.multi_step import _atgf
    from spikingjelly_b200.activation_based.cuda_kernel.neuron_kernel.single_step import lif as SL
    torch.manual_seed(0)
    sg = surrogate.ATan()
    T, N = 6, 257
    x0 = (torch.rand(T, N, device="cuda") * 2.5)
    gs, gv = torch.randn(T, N, device="cuda"), torch.randn(T, N, device="cuda") * 0.1

    def eager(step, extra=()):
        x = x0.clone().requires_grad_(True)
        v = torch.zeros(N, device="cuda", requires_grad=True)
        vv, ss, vs = v, [], []
        for t in range(T):
            s, vv = step(x[t], vv)
            ss.append(s)
            vs.append(vv)
        s_seq, v_seq = torch.stack(ss), torch.stack(vs)
        grads = torch.autograd.grad((s_seq * gs).sum() + (v_seq * gv).sum(), [x, v, *extra], allow_unused=True)
        return s_seq, v_seq, grads

    def check(run, step, extra=()):
        x = x0.clone().requires_grad_(True)
        v = torch.zeros(N, device="cuda", requires_grad=True)
        s, vs, _ = run(x, v)
        want_s, want_v, want_g = eager(step, extra)
        assert torch.equal(s, want_s) and torch.allclose(vs, want_v, atol=1e-6)
        got = torch.autograd.grad((s * gs).sum() + (vs * gv).sum(), [x, v, *extra], allow_unused=True)
        for a, b in zip(got, want_g):
            assert torch.allclose(a, b, atol=2e-4, rtol=1e-4), (a - b).abs().max()
    for soft, detach in ((False, False), (True, True)):
        vr = None if soft else 0.0
        check(lambda x, v: MI.cupy_multistep_if_forward(x, v, 1.0, 0.0, soft, detach, sg),
              lambda x, v: functional.neuron.if_step(x, v, 1.0, vr, sg, detach))
        for di in (True, False):
            check(lambda x, v: ML.cupy_multistep_lif_forward(x, v, 1.0, 0.0, soft, detach, 0.5, di, sg),
                  lambda x, v: functional.neuron.lif_step(x, v, 2.0, di, 1.0, vr, sg, detach))
    w = torch.tensor(0.3, device="cuda", requires_grad=True)
    for di in (True, False):
        check(lambda x, v: MP.cupy_multistep_plif_forward(x, v, 1.0, 0.0, False, False, w.sigmoid(), di, sg),
              lambda x, v: functional.neuron.plif_step(x, v, w, di, 1.0, 0.0, sg, False), extra=(w,))

    # a custom neuron through the extension classes: h = 0.9 v + 0.5 x
    class FP(NeuronFPTTKernel):
        def neuronal_charge(self):
            return "h_seq[t] = 0.9f * v_v_seq[t] + 0.5f * x_seq[t];"

    class BP(NeuronBPTTKernel):
        def grad_h_next_to_v(self):
            return "const float grad_h_next_to_v = 0.9f;"

        def grad_h_to_x(self):
            return "const float grad_h_to_x = 0.5f;"

    def custom(xt, vv):
        h = 0.9 * vv + 0.5 * xt
        sp = sg(h - 1.0)
        return sp, h * (1 - sp)
    check(lambda x, v: (*_atgf.run(x, v, 1.0, 0.0, FP(True, "float"), BP(sg, True, False, "float")), None), custom)
    # single step
    x1 = x0[0].clone().requires_grad_(True)
    v1 = (torch.rand(N, device="cuda") * 0.5).requires_grad_(True)
    s1, vn, _ = SL.cupy_single_step_lif_forward(x1, v1, 1.0, 0.0, False, 0.5, True, sg)
    x2, v2 = x1.detach().clone().requires_grad_(True), v1.detach().clone().requires_grad_(True)
    s2, vn2 = functional.neuron.lif_step(x2, v2, 2.0, True, 1.0, 0.0, sg, False)
    assert torch.equal(s1, s2) and torch.allclose(vn, vn2, atol=1e-6)
    g1 = torch.autograd.grad((s1 * gs[0]).sum() + (vn * gv[0]).sum(), [x1, v1])
    g2 = torch.autograd.grad((s2 * gs[0]).sum() + (vn2 * gv[0]).sum(), [x2, v2])
    assert all(torch.allclose(a, b, atol=2e-4, rtol=1e-4) for a, b in zip(g1, g2))
