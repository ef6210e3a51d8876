"""`flash_attention` public operator (src/mlx_train_perf/attention/api.py:52-123, :281-413).

`softmax(scale * Q K^T + mask) V` with GQA (kv head = q head // group, contiguous) and an
optional packed-segment mask, forward and backward on the CUDA library.  Only O and the
row log-sum-exp L are saved for the backward; no (S, S) tensor is ever allocated.

Layouts follow the reference: q (B, Hq, N, D), k/v (B, Hkv, N, D), O like q, L (B, Hq, N)
fp32 natural-log LSE of the scaled masked scores.  The tensors may be arbitrary strided views
as long as the head_dim axis is contiguous (e.g. a (B, N, H, D) projection transposed).
"""
from __future__ import annotations

import ctypes as C

import torch

from mlx_train_perf_b200 import _lib
from mlx_train_perf_b200.attention.segments import PackedMask
from mlx_train_perf_b200.core.loss import device_status
from mlx_train_perf_b200.errors import AttentionInputError, UnsupportedAttentionError

_KERNEL_DTYPES = (torch.float32, torch.bfloat16)
_KERNEL_HEAD_DIMS = (64, 96, 128)

# Engagement counter (attention/api.py:49 of the reference).
VJP_CALLS: dict[str, int] = {}
_TC_IMPLS = ("tc", "tc1", "tc2", "tc2s", "tc2s3", "tc2s4", "tcg", "tcp")


def _validate_shapes(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> None:
    for name, arr in (("q", q), ("k", k), ("v", v)):
        if arr.ndim != 4:
            raise AttentionInputError(f"{name} must be 4-D (B, H, N, D); got shape {tuple(arr.shape)}")
    b_q, hq, n_q, d_q = q.shape
    b_k, hkv, n_k, d_k = k.shape
    b_v, hv, n_v, d_v = v.shape
    if b_q < 1:
        raise AttentionInputError(f"batch must be >= 1; got {b_q}")
    if not (b_q == b_k == b_v):
        raise AttentionInputError(f"batch mismatch: q={b_q}, k={b_k}, v={b_v}")
    if hkv != hv:
        raise AttentionInputError(f"k/v head-count mismatch: k has {hkv} heads, v has {hv}")
    if hkv < 1 or hq % hkv != 0:
        raise AttentionInputError(f"Hq={hq} must be a multiple of Hkv={hkv} for GQA grouping")
    if not (n_q == n_k == n_v):
        raise AttentionInputError(f"sequence length mismatch: q={n_q}, k={n_k}, v={n_v}")
    if not (d_q == d_k == d_v):
        raise AttentionInputError(f"head_dim mismatch: q={d_q}, k={d_k}, v={d_v}")


def resolve_attention_impl(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, impl: str = "auto",
                           causal: bool = True, segments: PackedMask | None = None) -> str:
    """Gate of the kernel path (attention/api.py:75-123): dtype in {fp32, bf16}, head_dim in
    {64, 96, 128}, causal only, segments imply causal.  Returns "tc" (tcgen05 kernels: bf16, every head_dim
    of the gate has its own instantiation) or "simt" (CUDA-core kernels: fp32, or on request); never falls
    back silently."""
    _validate_shapes(q, k, v)
    if segments is not None and not causal:
        raise UnsupportedAttentionError(
            "segments (packed attention) require causal=True (got causal=False); "
            "packing composes on top of the causal triangle.")
    if impl not in ("auto", "kernel", "simt") + _TC_IMPLS:
        raise AttentionInputError(
            f"unknown impl {impl!r}; expected one of 'auto', 'kernel', 'tc', 'tc1', 'tc2', 'tc2s', 'simt'")
    if not (q.dtype == k.dtype == v.dtype):
        raise AttentionInputError(f"q/k/v dtypes differ: {q.dtype}, {k.dtype}, {v.dtype}")
    if not (q.device == k.device == v.device):
        # the kernels get raw device addresses: a host tensor or one on another GPU must never reach them
        raise AttentionInputError(f"q/k/v must live on one device; got {q.device}, {k.device}, {v.device}")
    if q.dtype not in _KERNEL_DTYPES:
        raise UnsupportedAttentionError(f"the kernels only support fp32/bf16 (got {q.dtype}).")
    head_dim = q.shape[-1]
    if head_dim not in _KERNEL_HEAD_DIMS:
        raise UnsupportedAttentionError(
            f"the kernels only support head_dim in {_KERNEL_HEAD_DIMS} (got {head_dim}).")
    if not causal:
        raise UnsupportedAttentionError("the kernels only support causal=True (got causal=False).")
    tc_ok = q.dtype == torch.bfloat16
    if impl == "simt":
        return "simt"
    # "tc1" / "tc2" force the single-tile / two-tile forward kernel, "tc2s" the two-tile kernel with every
    # query block's key range split over two CTAs
    if impl in _TC_IMPLS:
        if not tc_ok:
            raise UnsupportedAttentionError("impl='tc' serves bf16 tensors; use impl='simt' for fp32.")
        return impl
    return "tc" if tc_ok else "simt"


def _non_overlapping(t: torch.Tensor) -> bool:
    """True when no two elements of the (B, H, N, D) view share storage: unit head_dim stride and, going
    up the other axes from the smallest stride, each stride at least the extent below it.  Expanded
    (stride 0) heads or batches fail this; the backward writes gradients through these strides, so an
    aliasing view would make different heads race on the same memory."""
    if t.stride(-1) != 1:
        return False
    extent = t.shape[-1]
    for size, stride in sorted(((t.shape[i], t.stride(i)) for i in range(3)), key=lambda p: p[1]):
        if size == 1:
            continue
        if stride < extent:
            return False
        extent = stride * size
    return True


def _inner_contig(t: torch.Tensor) -> torch.Tensor:
    return t if _non_overlapping(t) else t.contiguous()


def _tc_strides_ok(t: torch.Tensor) -> bool:
    return all(s % 8 == 0 for s in t.stride()[:3]) and t.data_ptr() % 16 == 0


def _attn_args(q, k, v, o, *, scale, segments, impl):
    a = _lib.AttnArgs()
    a.b, a.hq, a.s, a.d = q.shape
    a.hkv = k.shape[1]
    a.dtype = _lib.BF16 if q.dtype == torch.bfloat16 else _lib.F32
    for name, t in (("q_stride", q), ("k_stride", k), ("v_stride", v), ("o_stride", o)):
        arr = getattr(a, name)
        for i in range(3):
            arr[i] = t.stride(i)
    a.scale = float(scale)
    a.causal = 1
    if segments is not None:
        a.seg_id = segments.seg_id.data_ptr()
        a.seg_start = segments.seg_start.data_ptr()
    a.impl = _lib.IMPL["tc" if impl in _TC_IMPLS else impl]
    # "tcg" / "tcp": dK / dV CTAs that cover a whole GQA group / one q head each (the library picks by grid size)
    a.reserved = {"tc1": 1, "tc2": 2, "tc2s": 2 | (2 << 3), "tcp": 64, "tcg": 128}.get(impl, 0)
    if impl.startswith("tc2s") and len(impl) == 5:      # "tc2s3" / "tc2s4": three / four shares
        a.reserved = 2 | (int(impl[4]) << 3)
    return a


def check_segment_contract(seg_id: torch.Tensor, seg_start: torch.Tensor) -> None:
    """The PackedMask contract the tensor-core kernels rely on (attention/segments.py:8-19 of the
    reference): per row, ids start at 0 and never decrease or skip, and seg_start[i] is the first index
    carrying seg_id[i].  The kernels decide block skipping and per-block masking from the ENDS of a
    tile, which is exact only under this contract.  Raises `AttentionInputError`; runs on whatever
    device the tensors live on (one host sync when that is a GPU)."""
    sid, sst = seg_id.to(torch.int64), seg_start.to(torch.int64)
    if sid.ndim != 2 or sid.shape != sst.shape:
        raise AttentionInputError("seg_id / seg_start must both be (B, N)")
    n = sid.shape[1]
    step = sid[:, 1:] - sid[:, :-1]
    idx = torch.arange(n, device=sid.device)[None].expand_as(sid)
    first = torch.where(torch.cat([torch.ones_like(sid[:, :1], dtype=torch.bool), step != 0], dim=1), idx,
                        torch.zeros_like(idx)).cummax(dim=1).values
    ok = bool((sid[:, 0] == 0).all()) and bool(((step == 0) | (step == 1)).all()) and bool((sst == first).all())
    if not ok:
        raise AttentionInputError(
            "segments violate the PackedMask contract: seg_id must start at 0 and rise by at most 1 along a "
            "row, and seg_start[i] must be the first index of segment seg_id[i]")


def _prep_segments(segments: PackedMask | None, b: int, n: int, device, validate: bool = False) -> PackedMask | None:
    if segments is None:
        return None
    sid, sst = segments.seg_id, segments.seg_start
    if tuple(sid.shape) != (b, n) or tuple(sst.shape) != (b, n):
        raise AttentionInputError(
            f"seg_id/seg_start must be (B, N) = ({b}, {n}); got {tuple(sid.shape)}, {tuple(sst.shape)}")
    if validate:
        check_segment_contract(sid, sst)
    sid = sid.to(device=device, dtype=torch.int32).contiguous()
    sst = sst.to(device=device, dtype=torch.int32).contiguous()
    return PackedMask(seg_id=sid, seg_start=sst)


def flash_fwd_raw(q, k, v, *, scale: float, segments: PackedMask | None = None, impl: str = "auto"):
    """(O, L) on the current stream."""
    lib = _lib.load()
    dev = q.device
    b, hq, n, d = q.shape
    o = torch.empty((b, hq, n, d), dtype=q.dtype, device=dev)
    lse = torch.empty((b, hq, n), dtype=torch.float32, device=dev)
    a = _attn_args(q, k, v, o, scale=scale, segments=segments, impl=impl)
    # scratch for the split over keys a small grid gets (0 bytes for most shapes)
    nbytes = lib.b200tp_flash_fwd_workspace_bytes(C.byref(a))
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev) if nbytes else None
    with torch.cuda.device(dev):
        rc = lib.b200tp_flash_fwd_ws(C.byref(a), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                                     lse.data_ptr(), ws.data_ptr() if nbytes else None, nbytes,
                                     torch.cuda.current_stream(dev).cuda_stream, device_status(dev).data_ptr())
    _lib.check(rc)
    return o, lse


def flash_fwd_workspace_bytes(q, k, v, *, scale: float, segments: PackedMask | None = None, impl: str = "auto") -> int:
    """Scratch bytes `flash_fwd_raw` will allocate for these tensors: non-zero exactly when the forward
    is split over keys (a small grid of long sequences), which also adds the combine kernel's launch."""
    a = _attn_args(q, k, v, q, scale=scale, segments=segments, impl=impl)
    return int(_lib.load().b200tp_flash_fwd_workspace_bytes(C.byref(a)))


def flash_bwd_workspace_bytes(q, k, v, *, scale: float, segments: PackedMask | None = None, impl: str = "auto") -> int:
    """Scratch bytes `flash_bwd_raw` will allocate: the row statistics (32 bytes per query row), plus the fp32
    per-q-head dK / dV partials when GQA heads get separate CTAs (small grids), which also adds the reduce
    kernel's launch."""
    a = _attn_args(q, k, v, q, scale=scale, segments=segments, impl=impl)
    return int(_lib.load().b200tp_flash_bwd_workspace_bytes(C.byref(a)))


_BWD_PARTS = {"all": 0, "dq": 256, "dkv": 512, "stats": 256 | 512}


def flash_bwd_raw(q, k, v, o, lse, d_o, *, scale: float, segments: PackedMask | None = None, impl: str = "auto",
                  parts: str = "all"):
    """(dQ, dK, dV) from saved O and L on the current stream.  `parts` other than "all" is for timing one
    kernel of the tensor-core backward alone: "dq" / "dkv" run the row-statistics pre-pass and only that
    kernel, "stats" only the pre-pass; the outputs of the kernels left out are returned unwritten."""
    lib = _lib.load()
    dev = q.device
    # d_o shares o's strides in the C ABI: bring it to o's layout if it differs.
    if d_o.stride() != o.stride():
        d_o = d_o.contiguous() if o.is_contiguous() else torch.empty_like(o).copy_(d_o)
    dq = torch.empty_strided(q.shape, q.stride(), dtype=q.dtype, device=dev)
    dk = torch.empty_strided(k.shape, k.stride(), dtype=k.dtype, device=dev)
    dv = torch.empty_strided(v.shape, v.stride(), dtype=v.dtype, device=dev)
    a = _attn_args(q, k, v, o, scale=scale, segments=segments, impl=impl)
    nbytes = lib.b200tp_flash_bwd_workspace_bytes(C.byref(a))
    a.reserved |= _BWD_PARTS[parts]
    ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        rc = lib.b200tp_flash_bwd(C.byref(a), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                                  lse.data_ptr(), d_o.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                  ws.data_ptr(), ws.numel(), torch.cuda.current_stream(dev).cuda_stream,
                                  device_status(dev).data_ptr())
    _lib.check(rc)
    return dq, dk, dv


class _FlashAttention(torch.autograd.Function):
    """(q, k, v[, seg_id, seg_start]) -> (O, L): L is a real output, never a captured stash
    (attention/api.py:8-12), and is marked non-differentiable."""

    @staticmethod
    def forward(ctx, q, k, v, seg_id, seg_start, scale, impl):
        segments = None if seg_id is None else PackedMask(seg_id=seg_id, seg_start=seg_start)
        o, lse = flash_fwd_raw(q, k, v, scale=scale, segments=segments, impl=impl)
        ctx.save_for_backward(q, k, v, o, lse, *([] if seg_id is None else [seg_id, seg_start]))
        ctx.scale = scale
        ctx.impl = impl
        ctx.mark_non_differentiable(lse)
        return o, lse

    @staticmethod
    def backward(ctx, d_o, _d_l):
        VJP_CALLS["flash_attention"] = VJP_CALLS.get("flash_attention", 0) + 1
        saved = ctx.saved_tensors
        q, k, v, o, lse = saved[:5]
        segments = PackedMask(seg_id=saved[5], seg_start=saved[6]) if len(saved) == 7 else None
        dq, dk, dv = flash_bwd_raw(q, k, v, o, lse, d_o.to(o.dtype), scale=ctx.scale, segments=segments,
                                   impl=ctx.impl)
        return dq, dk, dv, None, None, None, None


def flash_attention_with_lse(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale: float,
                             causal: bool = True, impl: str = "auto", segments: PackedMask | None = None,
                             validate_segments: bool = False):
    """(O, L).  See `flash_attention`."""
    resolved = resolve_attention_impl(q, k, v, impl=impl, causal=causal, segments=segments)
    if not q.is_cuda:
        raise AttentionInputError(f"q/k/v must be CUDA tensors (no CPU path); got {q.device}")
    q, k, v = _inner_contig(q), _inner_contig(k), _inner_contig(v)
    if resolved in _TC_IMPLS and not all(_tc_strides_ok(t) for t in (q, k, v)):
        if impl in _TC_IMPLS:
            raise UnsupportedAttentionError("impl='tc' needs 16-byte aligned tensors and strides")
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    seg = _prep_segments(segments, q.shape[0], q.shape[2], q.device, validate=validate_segments)
    return _FlashAttention.apply(q, k, v, None if seg is None else seg.seg_id,
                                 None if seg is None else seg.seg_start, float(scale), resolved)


def flash_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale: float, causal: bool = True,
                    impl: str = "auto", segments: PackedMask | None = None,
                    validate_segments: bool = False) -> torch.Tensor:
    """`softmax(scale * Q K^T + causal/segment mask) @ V` -> O (attention/api.py:281-413).

    `segments=PackedMask(seg_id, seg_start)` switches on block-diagonal-causal isolation: key
    j reaches query i iff same segment and j <= i.  Both passes run on the kernels; L stays an
    internal residual.

    The tensor-core kernels rely on the PackedMask contract (ids gapless and non-decreasing from 0
    along a row, seg_start consistent with them): they skip and mask whole key blocks from a tile's
    two ends.  A mask that breaks the contract gives results that differ from the per-element rule
    (and from impl="simt") without an error; `validate_segments=True` checks the contract first, at
    the price of one host synchronisation (like `validate_targets` of the loss)."""
    o, _ = flash_attention_with_lse(q, k, v, scale=scale, causal=causal, impl=impl, segments=segments,
                                    validate_segments=validate_segments)
    return o
