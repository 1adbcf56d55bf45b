"""Spiking self-attention kernel against the einsum definition in fp32."""
import pytest
import torch

from spikingjelly_b200.ops.ssa import ssa

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ref(S, L, H, scale):
    lead = S.shape[:-2]
    C = S.shape[-1] // 3
    q, k, v = S.float().reshape(-1, L, 3, H, C // H).unbind(2)       # [n, L, H, D]
    kv = torch.einsum("nlhd,nlhe->nhde", k, v)
    return (torch.einsum("nlhd,nhde->nlhe", q, kv) * scale).reshape(*lead, L, C)


@pytest.mark.parametrize("L,H,D", [(196, 8, 64), (49, 4, 32), (30, 2, 64)])
@pytest.mark.parametrize("binary", [True, False])
def test_ssa_forward_backward(L, H, D, binary):
    torch.manual_seed(0)
    T, B = 2, 3
    if binary:
        S = (torch.rand(T, B, L, 3 * H * D, device=DEV) < 0.2).to(torch.bfloat16)
    else:
        S = (torch.randn(T, B, L, 3 * H * D, device=DEV) * 0.5).to(torch.bfloat16)
    g = torch.randn(T, B, L, H * D, device=DEV).to(torch.bfloat16)
    Sa = S.clone().requires_grad_(True)
    out = ssa(Sa, L, H, 0.125)
    out.backward(g)
    Sr = S.float().requires_grad_(True)
    ref = _ref(Sr, L, H, 0.125)
    ref.backward(g.float())
    tol = dict(rtol=2e-2, atol=2e-2 * (L ** 0.5 if not binary else 1.0))
    torch.testing.assert_close(out.float(), ref, **tol)
    torch.testing.assert_close(Sa.grad.float(), Sr.grad, rtol=3e-2, atol=0.15 * (L ** 0.5 if not binary else 1.0) / 3)
    if binary:   # integer sums are exact in fp32 and representable in bf16 up to 256
        assert torch.equal(out.float(), ref.to(torch.bfloat16).float())
