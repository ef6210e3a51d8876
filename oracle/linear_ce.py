"""CPU oracle for the fused linear-cross-entropy path (TEST INFRASTRUCTURE ONLY).

Restates, in torch-CPU fp32 (or fp64 on request), the reference's
  * materialising loss           -- src/mlx_train_perf/core/naive.py:9-14
  * streaming LSE / target       -- src/mlx_train_perf/core/chunked.py:35-49
  * chunked backward to d_hidden -- src/mlx_train_perf/core/chunked.py:52-90
  * 4-bit affine group layout    -- src/mlx_train_perf/core/kernel/source.py:193-208
  * masked-mean reduction        -- src/mlx_train_perf/adapters/mlx_lm.py:212-215

`ignore_index` is not a reference concept: the reference masks rows outside the op
(adapters/mlx_lm.py:212-215).  Here an ignored row has NLL 0, target logit 0, zero
gradient and is excluded from `num_valid`; its LSE is still the true log-sum-exp.

The shipped operators never import this module.
"""
from __future__ import annotations

import math

import numpy as np
import torch

IGNORE_INDEX = -100


def _f(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    return x.detach().to(device="cpu", dtype=dtype)


# --------------------------------------------------------------------------------------
# int4 affine, group 64 along D (core/kernel/source.py:193-208; tests/test_quant_layout.py)
# --------------------------------------------------------------------------------------
def pack_int4(codes: torch.Tensor) -> torch.Tensor:
    """(V, D) integer codes in [0, 15] -> (V, D/8) words, low nibble first:
    `word[k >> 3] |= code[k] << 4 * (k & 7)`.  Returned as int32 holding the uint32 bits."""
    v, d = codes.shape
    assert d % 8 == 0
    c = codes.detach().cpu().numpy().astype(np.uint32).reshape(v, d // 8, 8)
    shifts = (4 * np.arange(8, dtype=np.uint32))[None, None, :]
    words = np.bitwise_or.reduce(c << shifts, axis=-1).astype(np.uint32)
    return torch.from_numpy(words.view(np.int32).copy())


def unpack_int4(w_q: torch.Tensor) -> torch.Tensor:
    """(V, D/8) words -> (V, D) int64 codes, nibble i of column k at bits [4i, 4i+4) of
    word k >> 3 with i = k & 7."""
    words = w_q.detach().cpu().numpy().view(np.uint32)
    v, nw = words.shape
    shifts = (4 * np.arange(8, dtype=np.uint32))[None, None, :]
    codes = (words[:, :, None] >> shifts) & np.uint32(0xF)
    return torch.from_numpy(codes.reshape(v, nw * 8).astype(np.int64))


def dequantize_int4(w_q: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor,
                    group_size: int = 64, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """`w = scale_g * code + bias_g` evaluated in fp32 (one fused multiply-add rounding is
    not modelled: scale*code is exact in fp32 for bf16 scales and 4-bit codes), then
    rounded ONCE to `out_dtype` (defaults to the scales' dtype).  This is the
    "fp32 dequant then round" contract the CUDA path follows; mx.dequantize evaluates in
    bf16 and rounds twice (tests/test_kernel_quant_parity.py:54-64)."""
    codes = unpack_int4(w_q).to(torch.float32)
    v, d = codes.shape
    s = _f(scales, torch.float32).repeat_interleave(group_size, dim=1)
    b = _f(biases, torch.float32).repeat_interleave(group_size, dim=1)
    assert s.shape == (v, d), (s.shape, (v, d))
    w = s * codes + b
    return w.to(out_dtype if out_dtype is not None else scales.dtype)


# --------------------------------------------------------------------------------------
# forward
# --------------------------------------------------------------------------------------
def naive_linear_ce(hidden: torch.Tensor, w: torch.Tensor, targets: torch.Tensor,
                    *, ignore_index: int = IGNORE_INDEX, dtype: torch.dtype = torch.float32):
    """(N,D) x (V,D) -> (nll, lse, tgt), each (N,) in `dtype`; materialises (N,V).

    Follows core/naive.py:9-14 on pre-upcast inputs (the reference's "fp32-exact" form)."""
    h = _f(hidden, dtype)
    ww = _f(w, dtype)
    t = targets.detach().cpu().to(torch.int64)
    logits = h @ ww.T
    lse = torch.logsumexp(logits, dim=-1)
    valid = t != ignore_index
    idx = torch.where(valid, t, torch.zeros_like(t))
    tgt = torch.take_along_dim(logits, idx[:, None], dim=-1).squeeze(-1)
    tgt = torch.where(valid, tgt, torch.zeros_like(tgt))
    nll = torch.where(valid, lse - tgt, torch.zeros_like(lse))
    return nll, lse, tgt


def streamed_lse_and_target(hidden: torch.Tensor, w: torch.Tensor, targets: torch.Tensor,
                            *, chunk_size: int = 8192, ignore_index: int = IGNORE_INDEX,
                            dtype: torch.dtype = torch.float32):
    """Online logaddexp over vocab chunks; never holds more than (N, chunk) logits.
    Follows core/chunked.py:35-49."""
    h = _f(hidden, dtype)
    t = targets.detach().cpu().to(torch.int64)
    n = h.shape[0]
    v = w.shape[0]
    lse = torch.full((n,), -math.inf, dtype=dtype)
    tgt = torch.zeros((n,), dtype=dtype)
    for v0 in range(0, v, chunk_size):
        v1 = min(v0 + chunk_size, v)
        logits = h @ _f(w[v0:v1], dtype).T
        lse = torch.logaddexp(lse, torch.logsumexp(logits, dim=-1))
        in_chunk = (t >= v0) & (t < v1)
        idx = torch.clamp(t - v0, 0, v1 - v0 - 1)
        got = torch.take_along_dim(logits, idx[:, None], dim=-1).squeeze(-1)
        tgt = torch.where(in_chunk, got, tgt)
    valid = t != ignore_index
    tgt = torch.where(valid, tgt, torch.zeros_like(tgt))
    nll = torch.where(valid, lse - tgt, torch.zeros_like(lse))
    return nll, lse, tgt


def shard_partials(hidden: torch.Tensor, w_shard: torch.Tensor, targets: torch.Tensor,
                   v_offset: int, *, dtype: torch.dtype = torch.float32):
    """Per-row (max, sum-exp relative to that max, target logit or 0) of one vocab shard
    `W[v_offset : v_offset + V_local]` -- the triple a vocab-sharded rank contributes."""
    h = _f(hidden, dtype)
    logits = h @ _f(w_shard, dtype).T
    m = logits.max(dim=-1).values
    s = torch.exp(logits - m[:, None]).sum(dim=-1)
    t = targets.detach().cpu().to(torch.int64) - v_offset
    inside = (t >= 0) & (t < w_shard.shape[0])
    idx = torch.clamp(t, 0, w_shard.shape[0] - 1)
    got = torch.take_along_dim(logits, idx[:, None], dim=-1).squeeze(-1)
    tgt = torch.where(inside, got, torch.zeros_like(got))
    return m, s, tgt


def combine_partials(ms, ss, ts, targets: torch.Tensor, *, ignore_index: int = IGNORE_INDEX):
    """Merge per-shard triples: m = max_r m_r, s = sum_r s_r e^{m_r-m}, lse = m + log s,
    tgt = sum_r t_r.  Returns (nll, lse, tgt)."""
    m = torch.stack(list(ms)).max(dim=0).values
    s = sum(si * torch.exp(mi - m) for mi, si in zip(ms, ss))
    lse = m + torch.log(s)
    tgt = sum(ts)
    valid = targets.detach().cpu().to(torch.int64) != ignore_index
    tgt = torch.where(valid, tgt, torch.zeros_like(tgt))
    nll = torch.where(valid, lse - tgt, torch.zeros_like(lse))
    return nll, lse, tgt


# --------------------------------------------------------------------------------------
# backward
# --------------------------------------------------------------------------------------
def chunked_backward(hidden: torch.Tensor, w: torch.Tensor, targets: torch.Tensor,
                     lse: torch.Tensor, cotangent: torch.Tensor, *, chunk_size: int = 8192,
                     ignore_index: int = IGNORE_INDEX, round_g_to: torch.dtype | None = None,
                     want_dw: bool = False, dtype: torch.dtype = torch.float32):
    """d_hidden (fp32, NOT cast down) and optionally d_w from the SAVED lse.

    Per chunk: p = exp(z - lse); g = (p - onehot) * ct; dH += g @ W_chunk;
    dW_chunk = g^T @ hidden (core/chunked.py:72-90).  `round_g_to` reproduces the
    reference rounding g to the weight dtype before the matmul (core/chunked.py:82-83);
    None keeps g in `dtype`.  Ignored rows get a zero cotangent."""
    h = _f(hidden, dtype)
    t = targets.detach().cpu().to(torch.int64)
    valid = t != ignore_index
    ct = _f(cotangent, dtype) * valid.to(dtype)
    ls = _f(lse, dtype)
    n, d = h.shape
    v = w.shape[0]
    dh = torch.zeros((n, d), dtype=dtype)
    dws = []
    for v0 in range(0, v, chunk_size):
        v1 = min(v0 + chunk_size, v)
        wc = _f(w[v0:v1], dtype)
        logits = h @ wc.T
        p = torch.exp(logits - ls[:, None])
        onehot = (torch.arange(v0, v1)[None, :] == t[:, None]).to(dtype)
        g = (p - onehot) * ct[:, None]
        if round_g_to is not None:
            g = g.to(round_g_to).to(dtype)
        dh += g @ wc
        if want_dw:
            dws.append(g.T @ h)
    return (dh, torch.cat(dws, dim=0)) if want_dw else (dh, None)


def masked_mean_cotangent(targets: torch.Tensor, *, ignore_index: int = IGNORE_INDEX):
    """Upstream gradient on the per-token NLL for loss = sum(nll * mask) / ntoks
    (adapters/mlx_lm.py:212-215): 1/num_valid on valid rows, 0 on ignored rows."""
    valid = targets.detach().cpu().to(torch.int64) != ignore_index
    nv = int(valid.sum())
    return valid.to(torch.float32) / max(nv, 1), nv
