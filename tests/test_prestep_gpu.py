"""Fused per-head RMSNorm + RoPE pre-step against a plain fp32 torch evaluation of the same formula
(the Hugging-Face / reference convention: y = n cos + rotate_half(n) sin, n = x rsqrt(mean x^2 + eps) w).

Tolerances: fp32 1e-5 of the largest value; bf16 one rounding of the fp32 result (half an ulp,
2^-9 relative) plus the rounding of the bf16 inputs to the gradient sums."""
import pytest
import torch

from mlx_train_perf_b200.attention.prestep import qk_norm_rope
from mlx_train_perf_b200.errors import AttentionInputError, UnsupportedAttentionError

pytestmark = pytest.mark.gpu


def _rotate_half(x):
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def _reference(x, cos, sin, weight, eps):
    x = x.double()
    n = x
    if weight is not None:
        n = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * weight.double()
    c, s = cos.double(), sin.double()
    if c.ndim == 2:
        c, s = c[None], s[None]
    return n * c.unsqueeze(-2) + _rotate_half(n) * s.unsqueeze(-2)


def _tables(length, d, dev, dtype, batch=None):
    inv = 1.0 / (10000.0 ** (torch.arange(0, d, 2, dtype=torch.float32, device=dev) / d))
    ang = torch.arange(length, dtype=torch.float32, device=dev)[:, None] * inv[None]
    emb = torch.cat((ang, ang), dim=-1)
    cos, sin = emb.cos().to(dtype), emb.sin().to(dtype)
    if batch is not None:
        cos, sin = cos[None].expand(batch, -1, -1).contiguous(), sin[None].expand(batch, -1, -1).contiguous()
    return cos, sin


@pytest.mark.parametrize("d", [64, 96, 128])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("norm", [True, False])
def test_forward_backward_parity(cuda_device, d, dtype, norm):
    dev = cuda_device
    torch.manual_seed(d + int(norm))
    b, length, h = 2, 37, 5
    x = torch.randn(b, length, h * d, device=dev).to(dtype).view(b, length, h, d).requires_grad_(True)
    w = (1 + 0.1 * torch.randn(d, device=dev)).to(dtype).requires_grad_(True) if norm else None
    cos, sin = _tables(length, d, dev, dtype, batch=b if d == 96 else None)
    g = torch.randn(b, length, h, d, device=dev).to(dtype)
    y = qk_norm_rope(x, cos, sin, weight=w, eps=1e-6)
    y.backward(g)
    xr = x.detach().clone().requires_grad_(True)
    wr = w.detach().clone().requires_grad_(True) if norm else None
    yr = _reference(xr, cos, sin, wr, 1e-6)
    yr.backward(g.double())
    tol = 1e-5 if dtype == torch.float32 else 6e-3
    assert (y.double() - yr).abs().max().item() <= tol * yr.abs().max().item()
    assert (x.grad.double() - xr.grad.double()).abs().max().item() <= tol * xr.grad.abs().max().item()
    if norm:
        gtol = 1e-5 if dtype == torch.float32 else 1.5e-2      # d_weight is rounded to bf16 once more
        assert (w.grad.double() - wr.grad.double()).abs().max().item() <= gtol * wr.grad.abs().max().item()


def test_transposed_consumer_and_refusals(cuda_device):
    dev = cuda_device
    x = torch.randn(1, 16, 4, 128, device=dev, dtype=torch.bfloat16)
    cos, sin = _tables(16, 128, dev, torch.bfloat16)
    y = qk_norm_rope(x, cos, sin)
    assert y.shape == x.shape and y.stride() == x.stride()
    assert y.transpose(1, 2).shape == (1, 4, 16, 128)          # consumed by flash_attention as a strided view
    with pytest.raises(UnsupportedAttentionError, match="head_dim"):
        qk_norm_rope(torch.randn(1, 4, 2, 80, device=dev), *_tables(4, 80, dev, torch.float32))
    with pytest.raises(AttentionInputError, match="cos"):
        qk_norm_rope(x, cos[:8], sin[:8])
    with pytest.raises(AttentionInputError, match="CUDA"):
        qk_norm_rope(x.cpu(), cos.cpu(), sin.cpu())
