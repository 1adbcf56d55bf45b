"""The allocation-free C entry point for BatchNorm statistics, called through its exported symbol.

Collected last on purpose (file name): it must pass both on its own and after every other GPU
test has used the library in the same process.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

OK, E_BAD_ARGUMENT, E_TOO_LARGE = 0, -1, -2
MAX_CHANNELS = 2048
DTYPE_CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


@pytest.fixture(scope="module")
def lib():
    from spikingjelly_b200 import ops
    ops.require()
    handle = ctypes.CDLL(str(ops.library_path()))
    fn = handle.sjb200_bn_stats_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                   ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    handle.sjb200_noalloc_last_error.restype = ctypes.c_char_p
    return handle


def _call(lib, y, gamma, beta, eps, outs):
    rows, channels = y.numel() // y.shape[-1], y.shape[-1]
    ptr = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())
    return lib.sjb200_bn_stats_noalloc(ptr(y), DTYPE_CODE[y.dtype], rows, channels, ptr(gamma), ptr(beta), eps,
                                       *[ptr(o) for o in outs], ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


@pytest.mark.parametrize("dtype,rows,channels", [(torch.bfloat16, 25088, 512), (torch.float32, 1000, 384),
                                                 (torch.float16, 77, 2048), (torch.bfloat16, 3, 8)])
def test_two_calls_in_a_row_match_the_regular_operator(lib, dtype, rows, channels):
    torch.manual_seed(rows + channels)
    dev = torch.device("cuda:0")
    gamma = torch.rand(channels, device=dev) + 0.5
    beta = torch.randn(channels, device=dev)
    outs = [torch.empty(channels, device=dev) for _ in range(4)]       # allocated before the calls under test
    inputs = [(torch.randn(rows, channels, device=dev) * s + m).to(dtype) for s, m in ((1.0, 0.0), (3.0, -2.0))]
    expected = [torch.ops.sjb200.bn_coefficients(y, gamma, beta, None, None, True, 0.1, 1e-5) for y in inputs]
    torch.cuda.synchronize()
    for y, want in zip(inputs, expected):                              # second call reuses the shared scratch
        before = torch.cuda.memory_allocated(dev)
        assert _call(lib, y, gamma, beta, 1e-5, outs) == OK, lib.sjb200_noalloc_last_error()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated(dev) == before
        for got, ref, name in zip(outs, want, ("mean", "invstd", "scale", "shift")):
            torch.testing.assert_close(got, ref, rtol=2e-5, atol=2e-6, msg=lambda m: f"{name}: {m}")


def test_without_affine_parameters(lib):
    y = torch.randn(4096, 64, device="cuda")
    outs = [torch.empty(64, device="cuda") for _ in range(4)]
    assert _call(lib, y, None, None, 1e-5, outs) == OK
    torch.cuda.synchronize()
    torch.testing.assert_close(outs[0], y.mean(0), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(outs[1], (y.var(0, unbiased=False) + 1e-5).rsqrt(), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(outs[2], outs[1])


def test_sizes_beyond_the_fixed_scratch_are_rejected(lib):
    channels = MAX_CHANNELS + 8
    y = torch.zeros(16, channels, device="cuda")
    outs = [torch.full((channels,), 7.0, device="cuda") for _ in range(4)]
    assert _call(lib, y, None, None, 1e-5, outs) == E_TOO_LARGE
    assert b"exceeds the fixed scratch capacity" in lib.sjb200_noalloc_last_error()
    torch.cuda.synchronize()
    assert all(bool((o == 7.0).all()) for o in outs)                   # nothing was launched
    y = torch.zeros(16, 12, device="cuda")
    assert _call(lib, y, None, None, 1e-5, [o[:12] for o in outs]) == E_BAD_ARGUMENT


def test_operands_that_are_not_device_memory_are_refused_before_any_launch(lib):
    """A host pointer (pageable or pinned) or a buffer of another device for ANY operand yields an error code and
    nothing is launched: a C or ctypes caller that passes the wrong buffer must not fault the device."""
    E_WRONG_DEVICE = -5
    y = torch.randn(256, 64, device="cuda")
    outs = [torch.full((64,), 7.0, device="cuda") for _ in range(4)]
    host = torch.zeros(64)
    pinned = torch.zeros(64).pin_memory()
    for bad_index in range(4):
        for bad in (host, pinned):
            trial = list(outs)
            trial[bad_index] = bad
            assert _call(lib, y, None, None, 1e-5, trial) == E_BAD_ARGUMENT
            assert b"not device memory" in lib.sjb200_noalloc_last_error()
    assert _call(lib, torch.randn(256, 64), None, None, 1e-5, outs) == E_BAD_ARGUMENT        # y on the host
    assert _call(lib, y, host, None, 1e-5, outs) == E_BAD_ARGUMENT                           # gamma on the host
    assert _call(lib, y, None, pinned, 1e-5, outs) == E_BAD_ARGUMENT                         # beta on the host
    if torch.cuda.device_count() > 1:
        other = torch.zeros(64, device="cuda:1")
        assert _call(lib, y, None, None, 1e-5, [other] + outs[1:]) == E_WRONG_DEVICE
        assert _call(lib, y, other, None, 1e-5, outs) == E_WRONG_DEVICE
    torch.cuda.synchronize()
    assert all(bool((o == 7.0).all()) for o in outs)                                         # nothing was launched
    assert _call(lib, y, None, None, 1e-5, outs) == OK                                       # and the entry point still works
    torch.cuda.synchronize()
    torch.testing.assert_close(outs[0], y.mean(0), rtol=1e-4, atol=1e-5)
