"""CPU oracle for causal / packed-segment GQA attention (TEST INFRASTRUCTURE ONLY).

Restates, in torch-CPU fp32 (or fp64 on request), the reference's
  * visibility rule        -- src/mlx_train_perf/attention/segments.py:22-29
  * GQA head mapping       -- src/mlx_train_perf/attention/reference.py:37-39
  * materialised forward   -- src/mlx_train_perf/attention/reference.py:42-116
  * hand-written backward  -- src/mlx_train_perf/attention/api.py:126-194

Layouts: q (B,Hq,N,D); k, v (B,Hkv,N,D); O like q; L (B,Hq,N) = natural-log LSE of the
scaled, masked scores.  Everything materialises (N,N): small N only.

The shipped operators never import this module.
"""
from __future__ import annotations

import math

import torch


def kv_head_for(q_head: int, group_size: int) -> int:
    """Contiguous GQA grouping: kv = q_head // group (attention/reference.py:37-39)."""
    return q_head // group_size


def segment_allowed(seg_id: torch.Tensor) -> torch.Tensor:
    """(B,1,N,N) bool: key j visible to query i iff same segment AND j <= i
    (attention/segments.py:22-29)."""
    sid = seg_id.detach().cpu()
    same = sid[:, None, :, None] == sid[:, None, None, :]
    n = sid.shape[-1]
    causal = torch.tril(torch.ones(n, n, dtype=torch.bool))[None, None]
    return same & causal


def _gather_kv(x: torch.Tensor, hq: int, hkv: int) -> torch.Tensor:
    group = hq // hkv
    idx = torch.tensor([kv_head_for(h, group) for h in range(hq)])
    return x.index_select(1, idx)


def _scores(q, k, *, scale: float, causal: bool, seg_id, dtype):
    hq, hkv = q.shape[1], k.shape[1]
    if hq % hkv != 0:
        raise ValueError(f"Hq={hq} must be a multiple of Hkv={hkv}")
    q32 = q.detach().cpu().to(dtype)
    kg = _gather_kv(k.detach().cpu().to(dtype), hq, hkv)
    s = (q32 @ kg.transpose(-1, -2)) * scale
    n = q.shape[2]
    if seg_id is not None:
        assert causal, "segments require causal=True"
        s = torch.where(segment_allowed(seg_id), s, torch.full_like(s, -math.inf))
    elif causal:
        mask = torch.triu(torch.ones(n, n, dtype=torch.bool), diagonal=1)
        s = s.masked_fill(mask, -math.inf)
    return s


def flash_attention_reference(q, k, v, *, scale: float, causal: bool = True, seg_id=None,
                              dtype: torch.dtype = torch.float32):
    """(O, L): O in `dtype` (NOT cast to the input dtype, so callers choose the rounding),
    L = logsumexp of the masked scaled scores (attention/reference.py:77-116)."""
    s = _scores(q, k, scale=scale, causal=causal, seg_id=seg_id, dtype=dtype)
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse[..., None])
    vg = _gather_kv(v.detach().cpu().to(dtype), q.shape[1], k.shape[1])
    return p @ vg, lse


def math_attention(q, k, v, *, scale: float, causal: bool = True, seg_id=None,
                   dtype: torch.dtype = torch.float32):
    """softmax(scale Q K^T + mask) V (attention/reference.py:93-103)."""
    return flash_attention_reference(q, k, v, scale=scale, causal=causal, seg_id=seg_id,
                                     dtype=dtype)[0]


def flash_attention_backward(q, k, v, o, lse, d_o, *, scale: float, causal: bool = True,
                             seg_id=None, dtype: torch.dtype = torch.float32):
    """(dQ, dK, dV) in `dtype` from saved O and L (attention/api.py:140-194):
    D = rowsum(dO*O); P = exp(S-L); dV = P^T dO; dP = dO V^T; dS = P*(dP-D);
    dQ = scale dS K; dK = scale dS^T Q; dK/dV summed over each kv head's q-head group."""
    b, hq, n, d = q.shape
    hkv = k.shape[1]
    group = hq // hkv
    q32 = q.detach().cpu().to(dtype)
    kg = _gather_kv(k.detach().cpu().to(dtype), hq, hkv)
    vg = _gather_kv(v.detach().cpu().to(dtype), hq, hkv)
    o32 = o.detach().cpu().to(dtype)
    do32 = d_o.detach().cpu().to(dtype)
    l32 = lse.detach().cpu().to(dtype)
    dd = (do32 * o32).sum(dim=-1)
    s = _scores(q, k, scale=scale, causal=causal, seg_id=seg_id, dtype=dtype)
    p = torch.exp(s - l32[..., None])
    dp = do32 @ vg.transpose(-1, -2)
    ds = p * (dp - dd[..., None])
    dq = scale * (ds @ kg)
    dv_h = p.transpose(-1, -2) @ do32
    dk_h = scale * (ds.transpose(-1, -2) @ q32)
    dv = dv_h.reshape(b, hkv, group, n, d).sum(dim=2)
    dk = dk_h.reshape(b, hkv, group, n, d).sum(dim=2)
    return dq, dk, dv


def bwd_D(d_o, o, dtype: torch.dtype = torch.float32):
    """D_i = sum_d dO_id O_id (attention/api.py:126-129)."""
    return (d_o.detach().cpu().to(dtype) * o.detach().cpu().to(dtype)).sum(dim=-1)


def segments_from_lengths(lengths, total: int | None = None):
    """seg_id / seg_start int32 (1, L) for consecutive segments of the given lengths
    (gapless, ascending ids from 0 -- the PackedMask contract, attention/segments.py:8-19)."""
    ids, starts = [], []
    cur = 0
    for i, n in enumerate(lengths):
        ids += [i] * n
        starts += [cur] * n
        cur += n
    if total is not None:
        assert cur == total, (cur, total)
    return (torch.tensor([ids], dtype=torch.int32), torch.tensor([starts], dtype=torch.int32))
