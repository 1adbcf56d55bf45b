"""Bit-operand GEMM, LIF/RMSNorm packers and the fused tensor-parallel sub-layer.  One GPU runs the same kernels on
local buffers; with two or more GPUs the ranks exchange bits and partial products through peer memory."""
import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _native_library():
    from spikingjelly_b200 import ops
    ops.require()


def _pack_rows(s: torch.Tensor, pitch: int) -> torch.Tensor:
    """[rows, C] {0,1} -> uint8 [rows, pitch], bit i of byte j = column 8j + i."""
    rows, C = s.shape
    b = s.to(torch.uint8).view(rows, C // 8, 8)
    w = (b << torch.arange(8, device=s.device, dtype=torch.uint8)).sum(-1).to(torch.uint8)
    out = torch.zeros(rows, pitch, dtype=torch.uint8, device=s.device)
    out[:, : C // 8] = w
    return out


def _unpack_rows(bits: torch.Tensor, C: int) -> torch.Tensor:
    sh = torch.arange(8, device=bits.device, dtype=torch.uint8)
    return ((bits[:, : C // 8, None] >> sh) & 1).reshape(bits.shape[0], -1).float()


@pytest.mark.parametrize("M,N,K", [(256, 256, 256), (1000, 768, 2048), (384, 136, 688), (4096, 2048, 768)])
def test_spike_gemm_local_matches_matmul(M, N, K):
    from spikingjelly_b200.parallel.fused_tp import pack_pitch
    torch.manual_seed(0)
    dev = "cuda"
    s = (torch.rand(M, K, device=dev) < 0.2).float()
    Kp = (K + 7) // 8 * 8
    sp = torch.zeros(M, Kp, device=dev)
    sp[:, :K] = s
    w = (torch.randn(N, K, device=dev) * 0.1).to(torch.bfloat16)
    wk = torch.zeros(N, (K + 7) // 8 * 8, dtype=torch.bfloat16, device=dev)
    wk[:, :K] = w
    pitch = pack_pitch(Kp)
    bits = _pack_rows(sp, pitch)
    out = torch.ops.sjb200.spike_gemm([bits.data_ptr()], pitch, M, K, wk, M, M, 0, [], 0)
    st = torch.ops.sjb200.gemm_status(out)
    assert st[0] == 0, st
    ref = s @ w.float().t()
    assert out.shape == (M, N) and (out.float() - ref).abs().max() <= 0.02 * ref.abs().max() + 1e-3


def test_lif_and_rmsnorm_packers_match_reference():
    from spikingjelly_b200.parallel.fused_tp import _lif_seq, pack_pitch
    torch.manual_seed(1)
    dev = "cuda"
    T, rows, C = 4, 300, 768
    x = (torch.randn(T, rows, C, device=dev) * 1.5).to(torch.bfloat16)
    pitch = pack_pitch(C)
    out = torch.zeros(T * rows, pitch, dtype=torch.uint8, device=dev)
    torch.ops.sjb200.lif_pack(x, out.data_ptr(), pitch, 2.0, 1.0)
    assert torch.equal(_unpack_rows(out, C), _lif_seq(x.float(), 2.0, 1.0).reshape(T * rows, C))
    for dtype in (torch.float32, torch.bfloat16):
        C = 2048
        h = (torch.randn(T, rows, C, device=dev) * 3).to(dtype)
        w = torch.rand(C, device=dev) + 0.5
        pitch = pack_pitch(C)
        out = torch.zeros(T * rows, pitch, dtype=torch.uint8, device=dev)
        torch.ops.sjb200.rmsnorm_lif_pack(h, w, [out.data_ptr()], pitch, 1e-6, 2.0, 1.0)
        hf = h.float()
        xn = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-6) * w
        ref = _lif_seq(xn, 2.0, 1.0).reshape(T * rows, C)
        got = _unpack_rows(out, C)
        assert (got != ref).float().mean() < 1e-4 and 0.01 < got.mean() < 0.6


def _sublayer_case(dev, T=4, tokens=512, d=512, F=1376, seed=0):
    g = torch.Generator().manual_seed(seed)
    h = (torch.randn(T, tokens, d, generator=g) * 2).to(dev)
    norm_w = (torch.rand(d, generator=g) + 1.5).to(dev)
    w1 = (torch.randn(F, d, generator=g) * 0.3).to(dev)
    w2 = (torch.randn(d, F, generator=g) * 0.05).to(dev)
    return h, norm_w, w1, w2


def _rel(a, b):
    return ((a - b).norm() / b.norm()).item()


def test_fused_sublayer_on_one_gpu_matches_reference():
    from spikingjelly_b200.parallel.fused_tp import FusedSpikingSubLayer, FusedTPWorkspace, _reference_sublayer
    dev = torch.device("cuda", 0)
    h, norm_w, w1, w2 = _sublayer_case(dev)
    ws = FusedTPWorkspace(T=4, tokens_per_rank=512, d_model=512, device=dev)
    layer = FusedSpikingSubLayer(ws, norm_w, w1, w2)
    for dtype in (torch.float32, torch.bfloat16):
        hh = h.to(dtype).clone()
        ref = _reference_sublayer(hh.float(), norm_w, w1, w2, 1e-6, 2.0, 1.0)
        delta_ref = ref - hh.float()
        assert delta_ref.abs().mean() > 1e-2
        out = layer(hh)
        ws.check()
        assert out.data_ptr() == hh.data_ptr()
        if dtype == torch.float32:
            assert _rel(out - h, delta_ref) < 0.03
        else:                                   # the sum itself is rounded to bf16: compare at the scale of h
            assert _rel(out.float(), ref) < 0.01


def _tp_worker(rank, world, init_file, out_dir):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"file://{init_file}", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from spikingjelly_b200.parallel.fused_tp import FusedSpikingSubLayer, FusedTPWorkspace, _reference_sublayer
    dev = torch.device("cuda", rank)
    T, tpr, d, F = 4, 256, 512, 1376
    h, norm_w, w1, w2 = _sublayer_case(dev, T, tpr * world, d, F)
    ws = FusedTPWorkspace(T=T, tokens_per_rank=tpr, d_model=d, device=dev)
    layer = FusedSpikingSubLayer(ws, norm_w, w1, w2)
    ref = _reference_sublayer(h, norm_w, w1, w2, 1e-6, 2.0, 1.0)
    res = {}
    for it in range(3):                                               # repeated calls reuse the buffers and advance the epoch
        mine = h[:, rank * tpr:(rank + 1) * tpr].contiguous()
        out = layer(mine)
        ws.check()
        want = ref[:, rank * tpr:(rank + 1) * tpr]
        res[f"rel_{it}"] = _rel(out - h[:, rank * tpr:(rank + 1) * tpr], want - h[:, rank * tpr:(rank + 1) * tpr])
    torch.save(res, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_sublayer_across_gpus_matches_reference():
    world = min(torch.cuda.device_count(), 4)
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_tp_worker, args=(world, os.path.join(d, "init"), d), nprocs=world, join=True)
        for r in range(world):
            res = torch.load(os.path.join(d, f"r{r}.pt"))
            assert res and max(res.values()) < 0.04, res
