"""Trainer loss shims for PyTorch (Hugging-Face style) Llama / Qwen2 / Qwen3 models: the
direct callers of the two operators (src/mlx_train_perf/adapters/mlx_lm.py:140-164
`split_model`, :167-216 `make_loss_fn`, :221-295 `make_packed_loss_fn`).

Both loss functions walk the inner model layer by layer --
`embed_tokens -> layers(h, mask) -> norm` -- so the mask each block sees is exactly "causal" or
a `PackedMask` (a top-level `model(input_ids)` call would hand the blocks a tensor mask, which
the flash wrapper refuses), then feed the hidden states to the fused loss with the logits never
materialised.  Masked mean: loss = sum(nll * mask) / ntoks, reduced inside the library.
"""
from __future__ import annotations

from typing import Any, Callable

import torch

from mlx_train_perf_b200.attention.segments import PackedMask
from mlx_train_perf_b200.attention.wrapper import SUPPORTED_FAMILIES, FlashAttentionWrapper
from mlx_train_perf_b200.core.loss import (IGNORE_INDEX, DenseHead, HeadRef, QuantizedHead,
                                           reduced_linear_cross_entropy, resolve_impl, tied_head)
from mlx_train_perf_b200.errors import AdapterError


def _head_from_module(mod: Any) -> HeadRef:
    """A `nn.Linear`-like lm_head -> DenseHead; a module carrying the 4-bit affine layout
    (`w_q` / `scales` / `biases` [, `group_size`, `bits`]) -> QuantizedHead."""
    if all(hasattr(mod, a) for a in ("w_q", "scales", "biases")):
        return QuantizedHead(w_q=mod.w_q, scales=mod.scales, biases=mod.biases,
                             group_size=int(getattr(mod, "group_size", 64)), bits=int(getattr(mod, "bits", 4)))
    w = getattr(mod, "weight", None)
    if isinstance(w, torch.Tensor) and w.ndim == 2:
        if getattr(mod, "bias", None) is not None:
            raise AdapterError("lm_head with a bias is not supported by the fused loss")
        return DenseHead(weight=w, trainable=bool(w.requires_grad))
    raise AdapterError(f"unsupported lm_head module type {type(mod).__name__!r}")


def split_model(model: Any) -> tuple[Callable[[torch.Tensor], torch.Tensor], HeadRef]:
    """(hidden-state trunk, HeadRef) of a causal-LM model; `AdapterError` for other shapes."""
    family = getattr(getattr(model, "config", None), "model_type", None)
    if family not in SUPPORTED_FAMILIES:
        raise AdapterError(f"unsupported model architecture (model_type {family!r}); supported: "
                           + ", ".join(SUPPORTED_FAMILIES))
    inner = getattr(model, "model", None)
    if inner is None or not all(hasattr(inner, a) for a in ("embed_tokens", "layers", "norm")):
        raise AdapterError("model.model must expose embed_tokens / layers / norm")
    if getattr(model.config, "tie_word_embeddings", False):
        w = inner.embed_tokens.weight
        head: HeadRef = tied_head(w, trainable=bool(w.requires_grad))
    else:
        head = _head_from_module(model.lm_head)

    def trunk(input_ids: torch.Tensor) -> torch.Tensor:
        return _walk(inner, input_ids, "causal")

    return trunk, head


def _walk(inner: Any, input_ids: torch.Tensor, mask: Any) -> torch.Tensor:
    h = inner.embed_tokens(input_ids)
    b, length = input_ids.shape
    pos = torch.arange(length, device=input_ids.device)[None].expand(b, -1)   # never reset per segment
    rope = inner.rotary_emb(h, pos) if hasattr(inner, "rotary_emb") else None
    for layer in inner.layers:
        out = layer(h, attention_mask=mask, position_ids=pos, position_embeddings=rope)
        h = out[0] if isinstance(out, tuple) else out
    return inner.norm(h)


def _require_wrapped(model: Any, who: str) -> None:
    for i, layer in enumerate(model.model.layers):
        if not isinstance(layer.self_attn, FlashAttentionWrapper):
            raise AdapterError(f"{who} requires enable_flash_attention(model) first; layer {i} self_attn is "
                               f"{type(layer.self_attn).__name__!r}")


def make_loss_fn(model: Any, *, impl: str = "auto"):
    """`loss(model, batch, lengths) -> (loss, ntoks)`: batch int (B, L+1); lengths int (B, 2)
    = (offset, length) per row; position s (1-based, on the target axis) is supervised iff
    offset <= s <= length."""
    split_model(model)
    _require_wrapped(model, "make_loss_fn")

    def loss_fn(model_arg: Any, batch: torch.Tensor, lengths: torch.Tensor):
        trunk, head = split_model(model_arg)
        inputs, targets = batch[:, :-1], batch[:, 1:]
        hidden = trunk(inputs)
        resolve_impl(head=head, dtype=hidden.dtype, n=hidden.shape[0] * hidden.shape[1], d=hidden.shape[-1],
                     impl=impl)
        steps = torch.arange(1, targets.shape[1] + 1, device=targets.device)
        mask = (steps >= lengths[:, 0:1]) & (steps <= lengths[:, 1:2])
        masked_targets = torch.where(mask, targets.to(torch.int64), torch.full_like(targets, IGNORE_INDEX,
                                                                                     dtype=torch.int64))
        # the masked mean (and the token count) are formed inside the library: unsupervised positions carry
        # ignore_index, so loss = sum(nll over supervised positions) / ntoks
        loss, count = reduced_linear_cross_entropy(hidden, head, masked_targets, impl=impl, reduction="mean")
        return loss, count.to(torch.int64)

    return loss_fn


def make_packed_loss_fn(model: Any, *, impl: str = "auto"):
    """`loss(model, batch, seg_id, seg_start, loss_mask) -> (loss, ntoks)` for the 4-tuple
    `packed_iterate_batches` yields; every block gets `PackedMask(seg_id, seg_start)`."""
    split_model(model)
    _require_wrapped(model, "make_packed_loss_fn")

    def loss_fn(model_arg: Any, batch: torch.Tensor, seg_id: torch.Tensor, seg_start: torch.Tensor,
                loss_mask: torch.Tensor):
        _, head = split_model(model_arg)
        inputs, targets = batch[:, :-1], batch[:, 1:]
        hidden = _walk(model_arg.model, inputs, PackedMask(seg_id=seg_id, seg_start=seg_start))
        masked_targets = torch.where(loss_mask, targets.to(torch.int64),
                                     torch.full_like(targets, IGNORE_INDEX, dtype=torch.int64))
        loss, count = reduced_linear_cross_entropy(hidden, head, masked_targets, impl=impl, reduction="mean")
        return loss, count.to(torch.int64)

    return loss_fn
