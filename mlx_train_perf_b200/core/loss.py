"""Fused, logit-free linear cross-entropy: public operator surface.

Mirrors src/mlx_train_perf/core/loss.py of the reference (head carriers :29-48, impl
resolution :51-123, validation :126-203, entry point :358-392) over torch tensors, with the
CUDA library behind it:

* `fused_linear_ce(hidden, head, targets)` returns the per-token `(nll, lse, target_logit)`
  triple -- the residual contract of the reference's inner custom function
  (core/loss.py:235-250) made public.  Only `nll` carries a gradient; the backward reads the
  SAVED `lse` and produces `d_hidden` in the hidden dtype with fp32 accumulation.
* `linear_cross_entropy(...)` applies `reduction` outside the op, as the reference does.

`ignore_index` rows are masked: NLL 0, no gradient, excluded from the `mean` denominator
(the masked mean of adapters/mlx_lm.py:212-215).  The (N, V) logits are never allocated.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Literal, Union

import torch

from mlx_train_perf_b200 import _lib
from mlx_train_perf_b200.errors import LossInputError, UnsupportedHeadError

IGNORE_INDEX = -100
_KERNEL_DTYPES = (torch.float32, torch.bfloat16)

# Engagement counters (the reference's VJP_CALLS, core/chunked.py:28-32): prove that the
# hand-written backward ran rather than autograd through some differentiable stand-in.
VJP_CALLS: dict[str, int] = {}


@dataclass(frozen=True)
class DenseHead:
    """`weight` (V, D) fp32/bf16; tied embeddings pass the same tensor.  `trainable` (default
    True, as in core/loss.py:29-33 of the reference) lets the backward also return d_weight when
    autograd asks for it (the weight requires grad); a frozen head (LoRA / QLoRA) costs
    nothing extra."""
    weight: torch.Tensor
    trainable: bool = True


@dataclass(frozen=True)
class QuantizedHead:
    """4-bit affine group-quantized head (frozen): `w_q` (V, D/8) int32/uint32 words holding
    8 codes each, low nibble first; `scales`, `biases` (V, D/group_size) bf16 or fp32;
    w = scale * code + bias (core/kernel/source.py:193-208)."""
    w_q: torch.Tensor
    scales: torch.Tensor
    biases: torch.Tensor
    group_size: int = 64
    bits: int = 4


HeadRef = Union[DenseHead, QuantizedHead]


def tied_head(embedding_weight: torch.Tensor, *, trainable: bool = False) -> DenseHead:
    return DenseHead(weight=embedding_weight, trainable=trainable)


# 4-bit heads on the tensor-core path: "tc_inline" expands the head inside the kernels whatever N is (no
# weight scratch), "tc_chunked" always dequantises chunk by chunk ahead of the dense kernels; plain "tc" /
# "auto" lets the library choose (the forward inside the kernel up to 512 rows, everything else chunked).
_TC_QUANT_IMPLS = ("tc_inline", "tc_chunked")
_QUANT_RESERVED = {"tc_inline": 0x10000, "tc_chunked": 0x20000}


@dataclass(frozen=True)
class Resolution:
    impl: Literal["tc", "simt", "tc_inline", "tc_chunked"]
    reason: str


def _quantized_head_d(head: QuantizedHead) -> int:
    return head.w_q.shape[-1] * (32 // head.bits)


def _require_kernel_supported(head: HeadRef, dtype: torch.dtype) -> None:
    if dtype not in _KERNEL_DTYPES:
        raise UnsupportedHeadError(
            f"the kernels only support fp32/bf16 hidden states (got {dtype}); cast the hidden states first.")
    if isinstance(head, QuantizedHead):
        if head.bits != 4:
            raise UnsupportedHeadError(f"only 4-bit quantized heads are supported (got bits={head.bits}).")
        if head.group_size != 64:
            raise UnsupportedHeadError(
                f"only group_size=64 quantized heads are supported (got group_size={head.group_size}).")
        d = _quantized_head_d(head)
        if d % 64 != 0:
            raise UnsupportedHeadError(
                f"a quantized head needs a hidden dim that is a multiple of 64 (got d={d}).")


def resolve_impl(*, head: HeadRef, dtype: torch.dtype, n: int, d: int | None = None,
                 impl: str = "auto") -> Resolution:
    """Pick the kernel family; never falls back silently (core/loss.py:94-123).

    "auto"/"kernel": tensor-core (tcgen05) kernels for bf16 with D % 8 == 0, CUDA-core
    kernels for fp32 (exact fp32 accumulation) and odd D.  "tc"/"simt" force one family and
    raise `UnsupportedHeadError` when it cannot serve the input."""
    if n <= 0:
        raise LossInputError(f"n must be positive (hidden's row count); got n={n}")
    if impl not in ("auto", "kernel", "tc", "simt") + _TC_QUANT_IMPLS:
        raise LossInputError(f"unknown impl {impl!r}; expected one of 'auto', 'kernel', 'tc', 'simt'")
    _require_kernel_supported(head, dtype)
    tc_ok = dtype == torch.bfloat16 and (d is None or d % 8 == 0)
    if impl == "simt":
        return Resolution("simt", "explicit impl='simt'")
    if impl == "tc" or impl in _TC_QUANT_IMPLS:
        if not tc_ok:
            raise UnsupportedHeadError(
                "impl='tc' needs bf16 operands and a hidden dim that is a multiple of 8; use impl='simt'.")
        if impl in _TC_QUANT_IMPLS and not isinstance(head, QuantizedHead):
            raise UnsupportedHeadError(f"impl={impl!r} selects how a 4-bit head is dequantised; this head is dense.")
        return Resolution(impl, f"explicit impl={impl!r}")
    if tc_ok:
        return Resolution("tc", "bf16 operands: tcgen05 kernels")
    return Resolution("simt", f"{dtype} operands: CUDA-core kernels with fp32 accumulation")


def _validate_inputs(hidden: torch.Tensor, head: HeadRef, targets: torch.Tensor, *,
                     validate_targets: bool, ignore_index: int) -> None:
    if hidden.ndim not in (2, 3):
        raise LossInputError(f"hidden must be 2D (N,D) or 3D (B,S,D), got shape {tuple(hidden.shape)}")
    leading = tuple(hidden.shape[:-1])
    n_total = 1
    for size in leading:
        n_total *= size
    if n_total <= 0:
        raise LossInputError(f"hidden must have at least one row, got leading dims {leading}")
    if tuple(targets.shape) != leading:
        raise LossInputError(f"targets shape {tuple(targets.shape)} must match hidden's leading dims {leading}")
    if targets.dtype.is_floating_point or targets.dtype == torch.bool or targets.dtype.is_complex:
        raise LossInputError(f"targets must be an integer dtype, got {targets.dtype}")
    d = hidden.shape[-1]
    if isinstance(head, DenseHead):
        if head.weight.ndim != 2 or head.weight.shape[-1] != d:
            raise LossInputError(
                f"head.weight's last dim ({head.weight.shape[-1]}) must match hidden's D ({d})")
        if hidden.dtype != head.weight.dtype:
            raise LossInputError(
                f"hidden dtype {hidden.dtype} must match dense head weight dtype {head.weight.dtype}")
        v = head.weight.shape[0]
    else:
        head_d = _quantized_head_d(head)
        if head_d != d:
            raise LossInputError(
                f"quantized head implies D={head_d} (from w_q shape and bits), which does not match hidden's D={d}")
        v = head.w_q.shape[0]
        if head.scales.shape != head.biases.shape or head.scales.shape[0] != v:
            raise LossInputError("scales/biases must both be (V, D/group_size)")
        if head.scales.dtype != head.biases.dtype or head.scales.dtype not in _KERNEL_DTYPES:
            raise LossInputError("scales/biases must share a dtype, fp32 or bf16")
    # Every operand is handed to the kernels as a raw device address: a tensor that lives on the host
    # (an offloaded or tied embedding, say) or on another GPU must be refused here, before any launch.
    operands = [("targets", targets)]
    if isinstance(head, DenseHead):
        operands.append(("head.weight", head.weight))
    else:
        operands += [("head.w_q", head.w_q), ("head.scales", head.scales), ("head.biases", head.biases)]
    for name, t in operands:
        if name == "targets" and not t.is_cuda:
            continue            # targets are moved with `.to(hidden.device)`: a host tensor is fine
        if t.device != hidden.device:
            raise LossInputError(
                f"{name} is on {t.device} but hidden is on {hidden.device}; every operand of the fused loss "
                "must live on the device the kernels run on (move it with .to(hidden.device))")
    if validate_targets:
        # One host sync; skip it on the training path with validate_targets=False.
        t = targets[targets != ignore_index]
        if t.numel() > 0:
            tmin, tmax = int(t.min()), int(t.max())
            if tmin < 0 or tmax >= v:
                raise LossInputError(
                    f"targets must satisfy 0 <= t < V={v} (or equal ignore_index={ignore_index}); "
                    f"got range [{tmin}, {tmax}]")


# ---------------------------------------------------------------------------------------
# native calls
# ---------------------------------------------------------------------------------------
_status: dict[int, torch.Tensor] = {}


def device_status(device: torch.device) -> torch.Tensor:
    """Per-device int32 word the kernels write when a bounded wait gives up."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _status:
        _status[idx] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
    return _status[idx]


def check_device_status(device: torch.device | None = None) -> None:
    """Synchronise and raise `DeviceTimeoutError` if any kernel reported a timed-out wait."""
    for idx, t in list(_status.items()):
        if device is not None and device.index is not None and idx != device.index:
            continue
        code = int(t.item())
        if code != 0:
            t.zero_()
            _lib.raise_for_device_status(code)


def _dtype_code(dt: torch.dtype) -> int:
    return _lib.BF16 if dt == torch.bfloat16 else _lib.F32


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _ce_args(hidden: torch.Tensor, head: HeadRef, targets: torch.Tensor, *, v_offset: int, ignore_index: int,
             impl: str) -> tuple[_lib.CeArgs, list]:
    keep: list = []
    a = _lib.CeArgs()
    a.hidden = hidden.data_ptr()
    a.targets = targets.data_ptr()
    a.n, a.d = hidden.shape
    a.dtype = _dtype_code(hidden.dtype)
    a.v_offset = v_offset
    a.ignore_index = ignore_index
    a.impl = _lib.IMPL["tc" if impl in _TC_QUANT_IMPLS else impl]
    a.reserved = _QUANT_RESERVED.get(impl, 0)
    if isinstance(head, DenseHead):
        w = head.weight.detach()
        if not w.is_contiguous():
            w = w.contiguous()
        keep.append(w)
        a.weight = w.data_ptr()
        a.v_local = w.shape[0]
        a.quant_bits = 0
        a.group_size = 0
        a.qparam_dtype = 0
    else:
        wq, sc, bi = head.w_q.contiguous(), head.scales.contiguous(), head.biases.contiguous()
        if wq.dtype not in (torch.int32, torch.uint32):
            raise LossInputError(f"w_q must hold 32-bit words (int32/uint32), got {wq.dtype}")
        keep += [wq, sc, bi]
        a.weight = None
        a.w_q, a.scales, a.biases = wq.data_ptr(), sc.data_ptr(), bi.data_ptr()
        a.v_local = wq.shape[0]
        a.quant_bits = head.bits
        a.group_size = head.group_size
        a.qparam_dtype = _dtype_code(sc.dtype)
    return a, keep


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _workspace(nbytes: int, device: torch.device) -> torch.Tensor | None:
    if nbytes == 0:
        return None
    return torch.empty(nbytes, dtype=torch.uint8, device=device)


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise LossInputError(f"{name} must be a CUDA tensor (the operators have no CPU path); got {t.device}")


def ce_forward_buffer(hidden: torch.Tensor, head: HeadRef, targets: torch.Tensor, *, v_offset: int = 0,
                      ignore_index: int = IGNORE_INDEX, impl: str = "auto", want_lse: bool = True) -> torch.Tensor:
    """One forward launch sequence over this call's vocab rows.

    Returns one (5, N) fp32 buffer: rows 0..2 are the (row_max, row_sumexp, tgt_logit) partial
    triple of these vocab rows (rows [0:3] are exactly the message a vocab-sharded rank
    contributes), rows 3..4 are lse and nll (left unwritten when `want_lse` is False)."""
    lib = _lib.load()
    dev = hidden.device
    n = hidden.shape[0]
    a, keep = _ce_args(hidden, head, targets, v_offset=v_offset, ignore_index=ignore_index, impl=impl)
    out = torch.empty((5, n), dtype=torch.float32, device=dev)
    nbytes = lib.b200tp_linear_ce_fwd_workspace_bytes(C.byref(a))
    ws = _workspace(nbytes, dev)
    with torch.cuda.device(dev):
        rc = lib.b200tp_linear_ce_fwd(
            C.byref(a), out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr(),
            out[3].data_ptr() if want_lse else None, out[4].data_ptr() if want_lse else None,
            _ptr(ws), nbytes, _stream(dev), device_status(dev).data_ptr())
    _lib.check(rc)
    del keep
    return out


def ce_forward_raw(hidden: torch.Tensor, head: HeadRef, targets: torch.Tensor, *, v_offset: int = 0,
                   ignore_index: int = IGNORE_INDEX, impl: str = "auto", want_lse: bool = True):
    """(row_max, row_sumexp, tgt_logit, lse, nll), each (N,) fp32; lse/nll are None when
    `want_lse` is False (vocab-sharded callers combine the triples across ranks first)."""
    out = ce_forward_buffer(hidden, head, targets, v_offset=v_offset, ignore_index=ignore_index, impl=impl,
                            want_lse=want_lse)
    return out[0], out[1], out[2], (out[3] if want_lse else None), (out[4] if want_lse else None)


def ce_backward_raw(hidden: torch.Tensor, head: HeadRef, targets: torch.Tensor, lse: torch.Tensor,
                    cotangent: torch.Tensor, *, v_offset: int = 0, ignore_index: int = IGNORE_INDEX,
                    impl: str = "auto", out_dtype: torch.dtype | None = None,
                    out: torch.Tensor | None = None, accumulate: bool = False,
                    d_weight: torch.Tensor | None = None) -> torch.Tensor:
    """d_hidden (N, D) from the saved lse.  `out_dtype=torch.float32` yields the fp32 partial a
    vocab-sharded caller reduces across ranks; `out` + `accumulate` adds into an fp32 buffer.
    `d_weight`: a contiguous (V_local, D) tensor of the weight dtype that receives g^T @ hidden
    (dense heads only; core/chunked.py:84-90)."""
    lib = _lib.load()
    dev = hidden.device
    n, d = hidden.shape
    a, keep = _ce_args(hidden, head, targets, v_offset=v_offset, ignore_index=ignore_index, impl=impl)
    odt = hidden.dtype if out_dtype is None else out_dtype
    if out is None:
        out = torch.empty((n, d), dtype=odt, device=dev)
    elif out.dtype != odt or tuple(out.shape) != (n, d) or not out.is_contiguous():
        raise LossInputError("out must be a contiguous (N, D) tensor of the requested dtype")
    lse = lse.to(torch.float32).contiguous()
    ct = cotangent.to(torch.float32).contiguous()
    nbytes = lib.b200tp_linear_ce_bwd_workspace_bytes(C.byref(a), _dtype_code(odt))
    ws = _workspace(nbytes, dev)
    if d_weight is not None:
        if not isinstance(head, DenseHead):
            raise UnsupportedHeadError("a quantized head is frozen: it has no d_weight")
        if (d_weight.dtype != head.weight.dtype or tuple(d_weight.shape) != tuple(head.weight.shape)
                or not d_weight.is_contiguous() or d_weight.device != dev):
            raise LossInputError("d_weight must be a contiguous tensor shaped and typed like the head weight")
    with torch.cuda.device(dev):
        if d_weight is None:
            rc = lib.b200tp_linear_ce_bwd(C.byref(a), lse.data_ptr(), ct.data_ptr(), out.data_ptr(),
                                          _dtype_code(odt), 1 if accumulate else 0, _ptr(ws), nbytes, _stream(dev),
                                          device_status(dev).data_ptr())
        else:
            rc = lib.b200tp_linear_ce_bwd_train(C.byref(a), lse.data_ptr(), ct.data_ptr(), out.data_ptr(),
                                                _dtype_code(odt), 1 if accumulate else 0, d_weight.data_ptr(),
                                                _ptr(ws), nbytes, _stream(dev), device_status(dev).data_ptr())
    _lib.check(rc)
    del keep
    return out


class _FusedLinearCE(torch.autograd.Function):
    """(hidden, targets) -> (nll, lse, tgt); the head is a constant (frozen)."""

    @staticmethod
    def forward(ctx, hidden, targets, head, ignore_index, impl):
        _, _, tgt, lse, nll = ce_forward_raw(hidden, head, targets, ignore_index=ignore_index, impl=impl)
        ctx.save_for_backward(hidden, targets, lse)
        ctx.head = head
        ctx.ignore_index = ignore_index
        ctx.impl = impl
        ctx.mark_non_differentiable(lse, tgt)
        return nll, lse, tgt

    @staticmethod
    def backward(ctx, g_nll, _g_lse, _g_tgt):
        key = "quantized" if isinstance(ctx.head, QuantizedHead) else "dense"
        VJP_CALLS[key] = VJP_CALLS.get(key, 0) + 1
        hidden, targets, lse = ctx.saved_tensors
        d_hidden = ce_backward_raw(hidden, ctx.head, targets, lse, g_nll, ignore_index=ctx.ignore_index,
                                   impl=ctx.impl)
        return d_hidden, None, None, None, None


class _FusedLinearCETrainable(torch.autograd.Function):
    """(hidden, weight, targets) -> (nll, lse, tgt) for a trainable dense head: the backward
    returns d_hidden and, when autograd needs it, d_weight (core/loss.py:235-262 of the
    reference: `_ce` with `head_trainable=True`)."""

    @staticmethod
    def forward(ctx, hidden, weight, targets, ignore_index, impl):
        head = DenseHead(weight=weight)
        _, _, tgt, lse, nll = ce_forward_raw(hidden, head, targets, ignore_index=ignore_index, impl=impl)
        ctx.save_for_backward(hidden, weight, targets, lse)
        ctx.ignore_index = ignore_index
        ctx.impl = impl
        ctx.mark_non_differentiable(lse, tgt)
        return nll, lse, tgt

    @staticmethod
    def backward(ctx, g_nll, _g_lse, _g_tgt):
        VJP_CALLS["dense_trainable"] = VJP_CALLS.get("dense_trainable", 0) + 1
        hidden, weight, targets, lse = ctx.saved_tensors
        d_w = torch.empty_like(weight, memory_format=torch.contiguous_format) if ctx.needs_input_grad[1] else None
        d_hidden = ce_backward_raw(hidden, DenseHead(weight=weight), targets, lse, g_nll,
                                   ignore_index=ctx.ignore_index, impl=ctx.impl, d_weight=d_w)
        return d_hidden, d_w, None, None, None


def _apply(hidden2, targets2, head, ignore_index, impl):
    """Route to the trainable form only when autograd will actually ask for d_weight."""
    if (isinstance(head, DenseHead) and head.trainable and head.weight.requires_grad
            and torch.is_grad_enabled()):
        w = head.weight if head.weight.is_contiguous() else head.weight.contiguous()
        return _FusedLinearCETrainable.apply(hidden2, w, targets2, ignore_index, impl)
    return _FusedLinearCE.apply(hidden2, targets2, head, ignore_index, impl)


class _FusedLinearCEReduced(torch.autograd.Function):
    """(hidden, weight | None, targets) -> (loss, count): the masked sum or mean of the per-row losses formed
    inside the library (one small kernel after the row combine, fixed summation order) instead of by a chain
    of eager reductions, and a backward whose cotangent vector comes from one small kernel fed with the
    upstream scalar and the saved count -- the masked mean of the reference's loss shim,
    adapters/mlx_lm.py:192-216, moved next to the operator.  `weight` is the dense weight when its gradient is
    wanted (then `head` is ignored), else None."""

    @staticmethod
    def forward(ctx, hidden, weight, targets, head, ignore_index, impl, mean):
        use = DenseHead(weight=weight) if weight is not None else head
        _, _, _, lse, nll = ce_forward_raw(hidden, use, targets, ignore_index=ignore_index, impl=impl)
        lib = _lib.load()
        dev = hidden.device
        out3 = torch.empty(3, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            rc = lib.b200tp_linear_ce_reduce(nll.data_ptr(), targets.data_ptr(), hidden.shape[0], ignore_index,
                                             out3.data_ptr(), _stream(dev))
        _lib.check(rc)
        saved = [hidden, targets, lse, out3] + ([weight] if weight is not None else [])
        ctx.save_for_backward(*saved)
        ctx.head, ctx.ignore_index, ctx.impl, ctx.mean = head, ignore_index, impl, mean
        loss, count = out3[1 if mean else 0], out3[2]
        ctx.mark_non_differentiable(count)
        return loss, count

    @staticmethod
    def backward(ctx, g_loss, _g_count):
        saved = ctx.saved_tensors
        hidden, targets, lse, out3 = saved[:4]
        weight = saved[4] if len(saved) == 5 else None
        head = DenseHead(weight=weight) if weight is not None else ctx.head
        key = "dense_trainable" if weight is not None else ("quantized" if isinstance(head, QuantizedHead) else "dense")
        VJP_CALLS[key] = VJP_CALLS.get(key, 0) + 1
        lib = _lib.load()
        dev = hidden.device
        n = hidden.shape[0]
        g = g_loss.to(torch.float32).reshape(1).contiguous()
        ct = torch.empty(n, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            rc = lib.b200tp_linear_ce_cotangent(targets.data_ptr(), n, ctx.ignore_index, g.data_ptr(),
                                                out3[2:].data_ptr() if ctx.mean else None, ct.data_ptr(), _stream(dev))
        _lib.check(rc)
        d_w = None
        if weight is not None and ctx.needs_input_grad[1]:
            d_w = torch.empty_like(weight, memory_format=torch.contiguous_format)
        d_hidden = ce_backward_raw(hidden, head, targets, lse, ct, ignore_index=ctx.ignore_index, impl=ctx.impl,
                                   d_weight=d_w)
        return d_hidden, d_w, None, None, None, None, None


def masked_loss(nll: torch.Tensor, targets: torch.Tensor, *, mean: bool = True,
                ignore_index: int = IGNORE_INDEX, upstream: torch.Tensor | None = None):
    """(loss, count, cotangent) of per-row losses that already exist (the vocab-sharded operator's
    replicated `nll`): the masked sum or mean and the valid-row count from one library kernel, and the
    per-row cotangent `upstream / count` (mean) or `upstream` (sum), zero on ignored rows, from another --
    the two launches `reduced_linear_cross_entropy` makes around its own forward and backward.
    `upstream` is a one-element fp32 device tensor (default 1)."""
    lib = _lib.load()
    dev = nll.device
    _require_cuda(nll, "nll")
    n = nll.shape[0]
    nll = nll.to(torch.float32).contiguous()
    targets = targets.reshape(-1).to(device=dev, dtype=torch.int64).contiguous()
    if targets.shape[0] != n:
        raise LossInputError(f"targets shape {tuple(targets.shape)} does not match nll shape {tuple(nll.shape)}")
    out3 = torch.empty(3, dtype=torch.float32, device=dev)
    ct = torch.empty(n, dtype=torch.float32, device=dev)
    g = torch.ones(1, dtype=torch.float32, device=dev) if upstream is None else upstream.to(torch.float32).reshape(1)
    with torch.cuda.device(dev):
        rc = lib.b200tp_linear_ce_reduce(nll.data_ptr(), targets.data_ptr(), n, ignore_index, out3.data_ptr(),
                                         _stream(dev))
        _lib.check(rc)
        rc = lib.b200tp_linear_ce_cotangent(targets.data_ptr(), n, ignore_index, g.data_ptr(),
                                            out3[2:].data_ptr() if mean else None, ct.data_ptr(), _stream(dev))
        _lib.check(rc)
    return out3[1 if mean else 0], out3[2], ct


def _apply_reduced(hidden2, targets2, head, ignore_index, impl, mean):
    trainable = (isinstance(head, DenseHead) and head.trainable and head.weight.requires_grad
                 and torch.is_grad_enabled())
    w = None
    if trainable:
        w = head.weight if head.weight.is_contiguous() else head.weight.contiguous()
    return _FusedLinearCEReduced.apply(hidden2, w, targets2, head, ignore_index, impl, mean)


def _prepare(hidden, head, targets, *, impl, validate_targets, ignore_index):
    _validate_inputs(hidden, head, targets, validate_targets=validate_targets, ignore_index=ignore_index)
    _require_cuda(hidden, "hidden")
    leading = tuple(hidden.shape[:-1])
    d = hidden.shape[-1]
    hidden2 = hidden.reshape(-1, d)
    if not hidden2.is_contiguous():
        hidden2 = hidden2.contiguous()
    targets2 = targets.reshape(-1).to(device=hidden.device, dtype=torch.int64).contiguous()
    res = resolve_impl(head=head, dtype=hidden2.dtype, n=hidden2.shape[0], d=d, impl=impl)
    return hidden2, targets2, leading, res


def fused_linear_ce(hidden: torch.Tensor, head: HeadRef, targets: torch.Tensor, *,
                    ignore_index: int = IGNORE_INDEX, impl: str = "auto", validate_targets: bool = False):
    """Per-token `(nll, lse, target_logit)`, each shaped like `targets`, fp32.

    hidden (N, D) or (B, S, D); targets integer, `ignore_index` rows masked.  Differentiable
    w.r.t. `hidden` through `nll` only."""
    hidden2, targets2, leading, res = _prepare(hidden, head, targets, impl=impl,
                                               validate_targets=validate_targets, ignore_index=ignore_index)
    nll, lse, tgt = _apply(hidden2, targets2, head, ignore_index, res.impl)
    return nll.reshape(leading), lse.reshape(leading), tgt.reshape(leading)


def linear_cross_entropy(hidden: torch.Tensor, head: HeadRef, targets: torch.Tensor, *,
                         impl: str = "auto", reduction: Literal["none", "mean", "sum"] = "mean",
                         ignore_index: int = IGNORE_INDEX, validate_targets: bool = True) -> torch.Tensor:
    """Cross-entropy of `hidden @ head^T` against `targets` without materialising logits
    (core/loss.py:358-392).  `mean` divides by the number of non-ignored rows (at least 1); `mean` and `sum`
    are reduced inside the library (see `_FusedLinearCEReduced`)."""
    if reduction not in ("none", "mean", "sum"):
        raise LossInputError(f"unknown reduction {reduction!r}; expected 'none', 'mean', or 'sum'")
    if reduction == "none":
        hidden2, targets2, leading, res = _prepare(hidden, head, targets, impl=impl,
                                                   validate_targets=validate_targets, ignore_index=ignore_index)
        nll, _, _ = _apply(hidden2, targets2, head, ignore_index, res.impl)
        return nll.reshape(leading)
    return reduced_linear_cross_entropy(hidden, head, targets, impl=impl, reduction=reduction,
                                        ignore_index=ignore_index, validate_targets=validate_targets)[0]


def reduced_linear_cross_entropy(hidden: torch.Tensor, head: HeadRef, targets: torch.Tensor, *,
                                 impl: str = "auto", reduction: Literal["mean", "sum"] = "mean",
                                 ignore_index: int = IGNORE_INDEX, validate_targets: bool = False):
    """`(loss, count)`: the masked `mean` (or `sum`) of the per-token losses and the number of rows whose
    target is not `ignore_index` (an fp32 scalar tensor, not differentiable) -- what a trainer's loss function
    returns as `(loss, ntoks)` (adapters/mlx_lm.py:192-216).  Nothing on this path synchronises with the host."""
    if reduction not in ("mean", "sum"):
        raise LossInputError(f"unknown reduction {reduction!r}; expected 'mean' or 'sum'")
    hidden2, targets2, _leading, res = _prepare(hidden, head, targets, impl=impl,
                                                validate_targets=validate_targets, ignore_index=ignore_index)
    return _apply_reduced(hidden2, targets2, head, ignore_index, res.impl, reduction == "mean")
