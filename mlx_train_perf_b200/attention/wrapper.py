"""`enable_flash_attention(model)`: swap every decoder layer's `self_attn` of a PyTorch
(Hugging-Face style) Llama / Qwen2 / Qwen3 model for a module that routes attention through
`flash_attention` (src/mlx_train_perf/attention/wrapper.py:72-157, :205-292).

The wrapper reproduces the stock attention exactly -- q/k/v projections, view as
(B, L, H, hd), optional per-head q/k RMSNorm (Qwen3), rotary embedding from the
`position_embeddings=(cos, sin)` pair, attention, `o_proj` -- replacing only the attention
call.  The (B, L, H, hd) projections are handed to the kernels as strided (B, H, L, hd) views, so
neither transpose is materialised.

The original submodules are kept as direct children under their original names
(`self_attn.q_proj`, ...): LoRA tooling that discovers targets by module path keeps working,
attribute lookup happens at call time (adapters injected later are used), and the parameters
stay registered.

Mask contract: `None` or the string "causal" mean plain causal; a `PackedMask` switches on
packed-segment attention; tensor masks (sliding-window / additive / padding) and KV caches are
refused -- this is a training-only, full-attention path.
"""
from __future__ import annotations

from typing import Any

import torch
from torch import nn

from mlx_train_perf_b200.attention.api import flash_attention
from mlx_train_perf_b200.attention.prestep import qk_norm_rope
from mlx_train_perf_b200.attention.segments import PackedMask
from mlx_train_perf_b200.errors import AttentionInputError, UnsupportedAttentionError

SUPPORTED_FAMILIES = ("llama", "qwen2", "qwen3")
KERNEL_HEAD_DIMS = (64, 96, 128)


def _resolve_mask(mask: Any) -> bool | PackedMask:
    """Map a call-time mask onto `flash_attention`'s arguments, or refuse."""
    if isinstance(mask, PackedMask):
        return mask
    if isinstance(mask, str):
        if mask == "causal":
            return True
        raise AttentionInputError(
            f"unsupported string mask {mask!r}; the flash-attention training path only supports the 'causal' mask")
    if mask is None:
        return True
    raise AttentionInputError(
        "tensor attention masks (sliding-window / additive / padding) are not supported; the flash-attention "
        "training path is causal-only -- pass None, 'causal' or a PackedMask")


def _rotate_half(x: torch.Tensor) -> torch.Tensor:
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def _norm_eps(norm: nn.Module) -> float:
    return float(getattr(norm, "variance_epsilon", None) or getattr(norm, "eps", None) or 1e-6)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x (B, L, H, hd); cos/sin (B, L, hd) or (L, hd) -- the Hugging-Face half-rotation form."""
    cos, sin = cos.unsqueeze(-2), sin.unsqueeze(-2)
    return (x * cos + _rotate_half(x) * sin).to(x.dtype)


class FlashAttentionWrapper(nn.Module):
    """Drop-in replacement for a Llama / Qwen2 / Qwen3 attention module."""

    def __init__(self, original: nn.Module, *, impl: str = "auto", head_dim: int | None = None,
                 n_heads: int | None = None, n_kv_heads: int | None = None) -> None:
        super().__init__()
        self.q_proj, self.k_proj = original.q_proj, original.k_proj
        self.v_proj, self.o_proj = original.v_proj, original.o_proj
        self._has_qk_norm = hasattr(original, "q_norm") and hasattr(original, "k_norm")
        if self._has_qk_norm:
            self.q_norm, self.k_norm = original.q_norm, original.k_norm
        cfg = getattr(original, "config", None)
        self.head_dim = int(head_dim or getattr(original, "head_dim", None)
                            or cfg.hidden_size // cfg.num_attention_heads)
        self.n_heads = int(n_heads or getattr(original, "num_heads", None) or cfg.num_attention_heads)
        self.n_kv_heads = int(n_kv_heads or getattr(original, "num_key_value_heads", None)
                              or getattr(cfg, "num_key_value_heads", self.n_heads))
        self.scale = float(getattr(original, "scaling", None) or self.head_dim ** -0.5)
        self.layer_idx = getattr(original, "layer_idx", None)
        self._impl = impl

    def forward(self, hidden_states: torch.Tensor, position_embeddings=None, attention_mask: Any = None,
                past_key_values: Any = None, past_key_value: Any = None, **_unused):
        if past_key_values is not None or past_key_value is not None:
            raise AttentionInputError("FlashAttentionWrapper is a training-only path; a KV cache is not supported")
        b, length, _ = hidden_states.shape
        q = self.q_proj(hidden_states).view(b, length, self.n_heads, self.head_dim)
        k = self.k_proj(hidden_states).view(b, length, self.n_kv_heads, self.head_dim)
        v = self.v_proj(hidden_states).view(b, length, self.n_kv_heads, self.head_dim)
        if position_embeddings is not None and q.is_cuda:
            # per-head RMSNorm (Qwen3) + RoPE as one kernel per tensor, on the projection's own layout
            cos, sin = position_embeddings
            qw, kw, q_eps, k_eps = None, None, 0.0, 0.0
            if self._has_qk_norm:
                qw, kw = self.q_norm.weight.to(q.dtype), self.k_norm.weight.to(k.dtype)
                q_eps, k_eps = _norm_eps(self.q_norm), _norm_eps(self.k_norm)
            q = qk_norm_rope(q, cos, sin, weight=qw, eps=q_eps)
            k = qk_norm_rope(k, cos, sin, weight=kw, eps=k_eps)
        else:
            if self._has_qk_norm:
                q, k = self.q_norm(q), self.k_norm(k)
            if position_embeddings is not None:
                cos, sin = position_embeddings
                q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        resolved = _resolve_mask(attention_mask)
        segments = resolved if isinstance(resolved, PackedMask) else None
        out = flash_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), scale=self.scale,
                              causal=True, segments=segments, impl=self._impl)        # (B, H, L, hd)
        out = out.transpose(1, 2).reshape(b, length, self.n_heads * self.head_dim)
        return self.o_proj(out), None


def _head_dim(config: Any) -> int:
    return int(getattr(config, "head_dim", None) or config.hidden_size // config.num_attention_heads)


def enable_flash_attention(model: Any, *, impl: str = "auto", seq_len: int | None = None, batch_size: int = 1,
                           packed: bool = False) -> None:
    """Enable the flash-attention training path on a model IN PLACE.

    Refuses (`UnsupportedAttentionError`) at enable time rather than mid-run: a model family
    other than Llama / Qwen2 / Qwen3; any non-"full_attention" entry in `config.layer_types` or
    an active sliding window; configured attention dropout; a head_dim outside {64, 96, 128}.

    `seq_len` / `batch_size` / `packed` are accepted for signature compatibility with the
    reference, whose kernels need a rate-cache pre-warm before a compiled step; these kernels
    have no calibration step, so the hints are unused."""
    del seq_len, batch_size, packed
    config = getattr(model, "config", None)
    family = getattr(config, "model_type", None)
    if family not in SUPPORTED_FAMILIES:
        raise UnsupportedAttentionError(
            f"unsupported model architecture (model_type {family!r}); enable_flash_attention supports: "
            + ", ".join(SUPPORTED_FAMILIES))
    layer_types = getattr(config, "layer_types", None)
    if layer_types is not None:
        offending = sorted({lt for lt in layer_types if lt != "full_attention"})
        if offending:
            raise UnsupportedAttentionError(
                "enable_flash_attention supports full-attention models only; model declares "
                f"non-full-attention layer_types {offending}")
    if getattr(config, "use_sliding_window", False) and getattr(config, "sliding_window", None):
        raise UnsupportedAttentionError(
            "enable_flash_attention supports full-attention models only; model has a sliding-window "
            "attention configuration")
    dropout = getattr(config, "attention_dropout", 0.0)
    if dropout:
        raise UnsupportedAttentionError(
            f"enable_flash_attention does not support attention dropout (attention_dropout={dropout}); it must be 0")
    hd = _head_dim(config)
    if hd not in KERNEL_HEAD_DIMS:
        raise UnsupportedAttentionError(
            f"enable_flash_attention supports head_dim in {KERNEL_HEAD_DIMS}; model has head_dim={hd}")
    for layer in model.model.layers:
        if isinstance(layer.self_attn, FlashAttentionWrapper):
            continue
        layer.self_attn = FlashAttentionWrapper(layer.self_attn, impl=impl, head_dim=hd,
                                                n_heads=config.num_attention_heads,
                                                n_kv_heads=getattr(config, "num_key_value_heads",
                                                                   config.num_attention_heads))
