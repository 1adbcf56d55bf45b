"""Native operators can be traced with fake tensors (no GPU needed: only the library's schemas are used)."""
import pytest
import torch
from torch._subclasses.fake_tensor import FakeTensorMode


def _load():
    from spikingjelly_b200 import ops
    try:
        ops.load()
    except Exception as e:          # library not built on this machine
        pytest.skip(f"native library unavailable: {e}")


def test_fake_shapes_of_native_operators():
    _load()
    with FakeTensorMode():
        a = torch.empty(256, 64, dtype=torch.bfloat16, device="cuda")
        b = torch.empty(128, 64, dtype=torch.bfloat16, device="cuda")
        assert torch.ops.sjb200.gemm_16bit(a, b, False, False, False, 0).shape == (256, 128)
        assert torch.ops.sjb200.gemm_16bit(a, b.t().contiguous(), False, True, True, 0).dtype == torch.float32
        q, inv = torch.ops.sjb200.fp8_quantize(a, False)
        assert q.dtype == torch.float8_e4m3fn and q.shape == a.shape and inv.shape == (1,)
        assert torch.ops.sjb200.gemm_fp8(q, torch.ops.sjb200.fp8_quantize(b, False)[0], None, False, 1).shape == (256, 128)
        assert torch.ops.sjb200.bit_pack(a).shape == (256 * 64 // 8,)
        assert torch.ops.sjb200.bit_unpack(torch.empty(16, dtype=torch.uint8, device="cuda"), 100, torch.float16).shape == (100,)
        qkv = torch.empty(4, 196, 3 * 512, dtype=torch.bfloat16, device="cuda")
        assert torch.ops.sjb200.ssa_forward(qkv, 196, 8, 0.125).shape == (4, 196, 512)


def test_flexsn_custom_ops_have_fake_implementations():
    from spikingjelly_b200.ops import flexsn as K
    if K.nvcc_path() is None:
        pytest.skip("nvcc not present")

    def core(x, v):
        h = v + x
        s = (h >= 1.0).to(h.dtype)
        return s, h * (1 - s)

    handle = K.register_kernel_handle(K.build_kernel(core, 1, 1, 1, training=False))
    with FakeTensorMode():
        x = torch.empty(5, 32, device="cuda")
        res = torch.ops.sjb200_flexsn.forward(handle, [x, torch.empty(32, device="cuda")], True)
    assert [tuple(r.shape) for r in res] == [(5, 32), (5, 32), (32,)]
    K.release_kernel_handle(handle)
    with pytest.raises(KeyError):
        K.lookup_kernel_handle(handle)
