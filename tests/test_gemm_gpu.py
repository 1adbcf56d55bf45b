"""tcgen05 GEMM against an fp32 PyTorch reference, for every operand layout, odd sizes,
split-K and the autograd wrapper."""
import pytest
import torch

from spikingjelly_b200.ops import gemm as G

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ref(a, b, a_mn, b_mn):
    A = a.float().t() if a_mn else a.float()
    B = b.float().t() if b_mn else b.float()
    return A @ B.t()


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 512), (1000, 264, 200), (392, 128, 1024), (77, 8, 72)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_layouts(a_mn, b_mn, M, N, K, dtype):
    torch.manual_seed(0)
    if (a_mn and M % 8) or (b_mn and N % 8) or ((not a_mn or not b_mn) and K % 8):
        pytest.skip("leading dimension must be a multiple of 8")
    a = torch.randn((K, M) if a_mn else (M, K), device=DEV).to(dtype)
    b = torch.randn((K, N) if b_mn else (N, K), device=DEV).to(dtype)
    out = G.gemm(a, b, a_mn, b_mn)
    G.check_status(out)
    ref = _ref(a, b, a_mn, b_mn)
    tol = 2e-2 if dtype is torch.bfloat16 else 4e-3
    torch.testing.assert_close(out.float(), ref, rtol=tol, atol=tol * K ** 0.5)


def test_binary_operand_is_exact():
    """Spike (0/1) activations times bf16 weights: products are exact, sums are fp32."""
    x = (torch.rand(512, 256, device=DEV) < 0.2).to(torch.bfloat16)
    w = torch.randn(384, 256, device=DEV).to(torch.bfloat16)
    out = G.gemm(x, w, out_f32=True)
    G.check_status(out)
    torch.testing.assert_close(out, x.float() @ w.float().t(), rtol=1e-5, atol=1e-4)


@pytest.mark.parametrize("split", [1, 2, 7])
def test_split_k(split):
    a = torch.randn(4096, 256, device=DEV).to(torch.bfloat16)      # [K, M]
    b = torch.randn(4096, 128, device=DEV).to(torch.bfloat16)      # [K, N]
    out = G.gemm(a, b, True, True, out_f32=True, split_k=split)
    G.check_status(out)
    torch.testing.assert_close(out, a.float().t() @ b.float(), rtol=1e-3, atol=5e-2)
    again = G.gemm(a, b, True, True, out_f32=True, split_k=split)
    assert torch.equal(out, again)       # deterministic reduction order


def test_linear_autograd():
    x = torch.randn(3, 100, 512, device=DEV).to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(264, 512, device=DEV) * 0.05).to(torch.bfloat16).requires_grad_(True)
    y = G.linear(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    G.check_status(y)
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    yr = xr @ wr.t()
    yr.backward(g.float())
    torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=5e-2)
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=2e-2, atol=5e-2)
    torch.testing.assert_close(w.grad.float(), wr.grad, rtol=2e-2, atol=2e-1)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (1000, 264, 200), (392, 128, 512), (6272, 1536, 512)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_epilogue_column_statistics(M, N, K, dtype):
    """Per-channel sum and sum of squares from the GEMM epilogue equal those of the stored 16-bit result, and the
    batch-norm coefficients built from them equal the ones of the stand-alone statistics kernel."""
    torch.manual_seed(1)
    x = torch.randn(M, K, device=DEV).to(dtype).requires_grad_(True)
    w = (torch.randn(N, K, device=DEV) * 0.1).to(dtype).requires_grad_(True)
    y, part = G.linear_with_stats(x, w)
    G.check_status(y)
    # 32-row slices; the two-CTA kernel rounds M up to 256-row tiles (the extra slices hold zeros)
    assert part.shape[0] in ((M + 127) // 128 * 4, (M + 255) // 256 * 8) and part.shape[1:] == (2, N) and not part.requires_grad
    torch.testing.assert_close(y.float(), G.gemm(x.detach(), w.detach()).float(), rtol=0, atol=0)
    yd = y.detach().double()
    torch.testing.assert_close(part[:, 0].double().sum(0), yd.sum(0), rtol=1e-5, atol=1e-3)
    torch.testing.assert_close(part[:, 1].double().sum(0), (yd * yd).sum(0), rtol=1e-5, atol=1e-3)
    if N % 8 == 0 and N <= 4096:
        a = torch.ops.sjb200.bn_coefficients_partial(part, M, None, None, None, None, 0.1, 1e-5)
        b = torch.ops.sjb200.bn_coefficients(y.detach(), None, None, None, None, True, 0.1, 1e-5)
        for u, v in zip(a, b):
            torch.testing.assert_close(u, v, rtol=1e-5, atol=1e-6)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    (xr @ wr.t()).backward(g.float())
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=2e-2, atol=5e-2)
    torch.testing.assert_close(w.grad.float(), wr.grad, rtol=2e-2, atol=3e-1)


@pytest.fixture
def pair_mode():
    G.require()
    prev = torch.ops.sjb200.gemm_set_pair_mode(2)          # force the two-CTA kernel on every shape it supports
    yield
    torch.ops.sjb200.gemm_set_pair_mode(prev)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 512), (1000, 264, 200), (6272, 1536, 512)])
def test_cta_pair_kernel_layouts(pair_mode, a_mn, b_mn, M, N, K):
    """The two-CTA (cta_group::2) kernel against fp32 matmul, every operand layout, ragged edges in M, N and K."""
    torch.manual_seed(0)
    a = torch.randn((K, M) if a_mn else (M, K), device=DEV).to(torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device=DEV).to(torch.bfloat16)
    out = G.gemm(a, b, a_mn, b_mn)
    G.check_status(out)
    torch.testing.assert_close(out.float(), _ref(a, b, a_mn, b_mn), rtol=2e-2, atol=2e-2 * K ** 0.5)


def test_cta_pair_kernel_statistics_and_determinism(pair_mode):
    torch.manual_seed(2)
    x = torch.randn(1500, 512, device=DEV).to(torch.bfloat16)
    w = (torch.randn(520, 512, device=DEV) * 0.1).to(torch.bfloat16)
    y, part = G.linear_with_stats(x, w)
    G.check_status(y)
    yd = y.double()
    torch.testing.assert_close(part[:, 0].double().sum(0), yd.sum(0), rtol=1e-5, atol=1e-3)
    torch.testing.assert_close(part[:, 1].double().sum(0), (yd * yd).sum(0), rtol=1e-5, atol=1e-3)
    torch.ops.sjb200.gemm_set_pair_mode(0)
    y1 = G.gemm(x, w)
    assert torch.equal(y, y1)            # same k order and rounding as the single-CTA kernel


@pytest.mark.parametrize("split", [0, 3])
def test_cta_pair_kernel_split_k_and_fp32_output(pair_mode, split):
    a = torch.randn(4096, 512, device=DEV).to(torch.bfloat16)      # [K, M]
    b = torch.randn(4096, 264, device=DEV).to(torch.bfloat16)      # [K, N]
    out = G.gemm(a, b, True, True, out_f32=True, split_k=split)
    G.check_status(out)
    torch.testing.assert_close(out, a.float().t() @ b.float(), rtol=1e-3, atol=5e-2)
    assert torch.equal(out, G.gemm(a, b, True, True, out_f32=True, split_k=split))
    out16 = G.gemm(a, b, True, True, split_k=split)
    torch.testing.assert_close(out16.float(), a.float().t() @ b.float(), rtol=2e-2, atol=1.5)
