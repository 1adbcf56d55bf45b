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


def test_every_native_operator_has_a_fake_and_shapes_follow_the_kernels():
    """Fakes exist for all ``sjb200::`` operators that produce tensors; their shapes are those the CUDA side allocates."""
    _load()
    import torch._library.simple_registry as registry
    schemas = [n for n in torch._C._dispatch_get_all_op_names() if n.startswith("sjb200::")]
    host_only = {"sjb200::gemm_status", "sjb200::gemm_set_pair_mode", "sjb200::scan_chunk"}
    missing = [n for n in schemas if n.split(".")[0] not in host_only and
               registry.singleton.find(n.split(".")[0]).fake_impl.kernel is None]
    assert not missing, missing
    with FakeTensorMode():
        dev = "cuda"
        x = torch.empty(6, 3, 64, dtype=torch.bfloat16, device=dev)
        spike, v_last, v_seq, packed, ckpt = torch.ops.sjb200.scan_forward(x, None, 0.0, None, 1, 2.0, 0.0, 0.0, 0.0, 1.0, 0.0, False,
                                                                          True, True, True)
        assert spike.shape == x.shape and v_last.shape == (3, 64) and v_seq.shape == x.shape
        assert packed.shape == (6, 6) and packed.dtype == torch.int32 and ckpt.shape == (0,)      # T = 6 -> one chunk of 8
        x8 = torch.empty(20, 128, dtype=torch.float8_e4m3fn, device=dev)
        s8, *_rest, ck = torch.ops.sjb200.scan_forward(x8, None, 0.0, None, 1, 2.0, 0.0, 0.0, 0.0, 1.0, 0.0, False, False, False, True)
        assert s8.dtype == torch.bfloat16 and ck.shape == (2, 128)
        gx, gvi, gr = torch.ops.sjb200.scan_backward(spike, None, None, x, None, 0.0, None, None, 1, 2.0, 0.0, 0.0, 0.0, 1.0, 0.0, False,
                                                     1, 2.0, 0.0, True, False)
        assert gx.shape == x.shape and gvi.numel() == 0 and gr.numel() == 0
        y = torch.empty(8, 100, 64, dtype=torch.bfloat16, device=dev)
        mean, invstd, scale, shift = torch.ops.sjb200.bn_coefficients(y, None, None, None, None, True, 0.1, 1e-5)
        assert mean.shape == (64,) and shift.dtype == torch.float32
        out, ck = torch.ops.sjb200.bn_lif_forward(y, scale, shift, None, 1, 2.0, 1.0, 0.0, False, 0.0, True)
        assert out.shape == y.shape and ck.shape == (1, 6400)
        dy, gg, gb = torch.ops.sjb200.bn_lif_backward(out, y, scale, shift, mean, invstd, None, ck, True, 1, 2.0, 1.0, 0.0, False, 0.0,
                                                      1, 2.0, 0.0, True)
        assert dy.shape == y.shape and gg.shape == (64,) and gb.shape == (64,)
        img = torch.empty(8, 15, 15, 64, dtype=torch.bfloat16, device=dev)
        sp, idx = torch.ops.sjb200.bn_pool_lif_forward(img, scale, shift, 4, False, 1, 2.0, 1.0, 0.0, False, 0.0)
        assert sp.shape == (4, 2, 8, 8, 64) and idx.shape == (8, 8, 8, 64) and idx.dtype == torch.uint8
        w = torch.empty(128, 3, 3, 64, dtype=torch.bfloat16, device=dev)
        rows, stats = torch.ops.sjb200.conv2d_nhwc_forward(img, w, [2, 2], [1, 1], [1, 1], True)
        assert rows.shape == (8 * 8 * 8, 128) and stats.shape == (16, 2, 128)
        assert torch.ops.sjb200.conv2d_nhwc_dgrad(rows, w, 15, 15, [2, 2], [1, 1]).shape == img.shape
        gw = torch.ops.sjb200.conv2d_nhwc_wgrad(img, rows, 3, 3, [2, 2], [1, 1], [1, 1])
        assert gw.shape == (128, 3, 3, 64) and gw.dtype == torch.float32
