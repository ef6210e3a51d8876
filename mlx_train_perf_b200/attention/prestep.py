"""Fused attention pre-step: per-head RMSNorm (optional) + rotary position embedding on the
projection's own (B, L, H, d) view -- no transpose, one read and one write of the tensor.

The reference's wrapper runs `mx.fast.rms_norm` per head and then `rope` between the q / k
projections and the attention operator (attention/wrapper.py:133-157); this is that pair as one
CUDA kernel each way, differentiable w.r.t. the input and the norm weight.  Rotation convention:
element j pairs with j + d/2 (`y = n cos + rotate_half(n) sin`), cos / sin given per position as
(L, d) or (B, L, d) rows, the form Hugging-Face rotary modules hand to attention layers.
"""
from __future__ import annotations

import ctypes as C

import torch

from mlx_train_perf_b200 import _lib
from mlx_train_perf_b200.errors import AttentionInputError, UnsupportedAttentionError

_DTYPES = (torch.float32, torch.bfloat16)


def _args(x: torch.Tensor, y: torch.Tensor, weight, eps: float, cos: torch.Tensor, sin: torch.Tensor):
    a = _lib.PrestepArgs()
    a.b, a.l, a.h, a.d = x.shape
    a.dtype = _lib.BF16 if x.dtype == torch.bfloat16 else _lib.F32
    for i in range(3):
        a.x_stride[i] = x.stride(i)
        a.y_stride[i] = y.stride(i)
    a.weight = None if weight is None else weight.data_ptr()
    a.eps = float(eps)
    a.cos, a.sin = cos.data_ptr(), sin.data_ptr()
    a.cs_dtype = _lib.BF16 if cos.dtype == torch.bfloat16 else _lib.F32
    if cos.ndim == 3:
        a.cs_stride_b = cos.stride(0) if cos.shape[0] > 1 else 0
        a.cs_stride_l = cos.stride(1)
    else:
        a.cs_stride_b, a.cs_stride_l = 0, cos.stride(0)
    return a


def _check(x, weight, cos, sin):
    if x.ndim != 4:
        raise AttentionInputError(f"x must be (B, L, H, d); got shape {tuple(x.shape)}")
    if not x.is_cuda:
        raise AttentionInputError(f"x must be a CUDA tensor (no CPU path); got {x.device}")
    if x.dtype not in _DTYPES:
        raise UnsupportedAttentionError(f"the pre-step kernels only support fp32/bf16 (got {x.dtype}).")
    b, length, _, d = x.shape
    if d not in (64, 96, 128):
        raise UnsupportedAttentionError(f"the pre-step kernels only support head_dim in (64, 96, 128) (got {d}).")
    if x.stride(3) != 1:
        raise AttentionInputError("the head_dim axis of x must be contiguous")
    if weight is not None and (weight.shape != (d,) or weight.dtype != x.dtype or not weight.is_contiguous()
                               or weight.device != x.device):
        raise AttentionInputError(f"norm weight must be a contiguous ({d},) tensor of x's dtype on x's device")
    for name, t in (("cos", cos), ("sin", sin)):
        if t.ndim not in (2, 3) or t.shape[-1] != d or t.shape[-2] != length or t.stride(-1) != 1:
            raise AttentionInputError(f"{name} must be (L, d) or (B, L, d) with a contiguous last axis; got "
                                      f"{tuple(t.shape)}")
        if t.ndim == 3 and t.shape[0] not in (1, b):
            raise AttentionInputError(f"{name} batch {t.shape[0]} does not match x batch {b}")
        if t.dtype not in _DTYPES or t.device != x.device:
            raise AttentionInputError(f"{name} must be an fp32/bf16 tensor on x's device")
    if cos.shape != sin.shape or cos.stride() != sin.stride() or cos.dtype != sin.dtype:
        raise AttentionInputError("cos and sin must share shape, strides and dtype")


class _NormRope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, cos, sin, eps):
        lib = _lib.load()
        y = torch.empty_like(x, memory_format=torch.preserve_format)
        a = _args(x, y, weight, eps, cos, sin)
        with torch.cuda.device(x.device):
            rc = lib.b200tp_qk_norm_rope_fwd(C.byref(a), x.data_ptr(), y.data_ptr(),
                                             torch.cuda.current_stream(x.device).cuda_stream)
        _lib.check(rc)
        ctx.save_for_backward(x, weight, cos, sin)
        ctx.eps = eps
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight, cos, sin = ctx.saved_tensors
        lib = _lib.load()
        if dy.stride(3) != 1:
            dy = dy.contiguous()
        dx = torch.empty_like(x, memory_format=torch.preserve_format)
        a = _args(x, dy, weight, ctx.eps, cos, sin)
        want_dw = weight is not None and ctx.needs_input_grad[1]
        dw = torch.empty(x.shape[-1], dtype=torch.float32, device=x.device) if want_dw else None
        nbytes = lib.b200tp_qk_norm_rope_bwd_workspace_bytes(C.byref(a)) if want_dw else 0
        ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=x.device) if want_dw else None
        with torch.cuda.device(x.device):
            rc = lib.b200tp_qk_norm_rope_bwd(C.byref(a), x.data_ptr(), dy.data_ptr(), dx.data_ptr(),
                                             None if dw is None else dw.data_ptr(),
                                             None if ws is None else ws.data_ptr(), nbytes,
                                             torch.cuda.current_stream(x.device).cuda_stream)
        _lib.check(rc)
        return dx, (None if dw is None else dw.to(weight.dtype)), None, None, None


def qk_norm_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, *, weight: torch.Tensor | None = None,
                 eps: float = 1e-6) -> torch.Tensor:
    """`rope(rms_norm(x) * weight)` over the last axis of x (B, L, H, d); `weight=None` skips the
    norm.  fp32 arithmetic, one rounding to x's dtype; output has x's strides."""
    _check(x, weight, cos, sin)
    if not x.is_contiguous():      # the projection's (B, L, H * d) output viewed per head is; odd views are copied
        x = x.contiguous()
    return _NormRope.apply(x, weight, cos, sin, float(eps))
