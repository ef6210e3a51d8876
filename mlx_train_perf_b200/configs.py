"""Seeded synthetic inputs for the five benchmark / parity configurations.

Everything is drawn in fp32 from one `torch.Generator` per config in a fixed order and cast
afterwards, so a CPU checker and the GPU path can be fed bit-identical tensors (generate on
CPU, then copy).  `device="cuda"` draws on the GPU instead (fast, used by the benchmark when
no element-wise comparison with a CPU run is wanted); the two streams differ.

  C1  N=2048  D=1024 V=32768  fp32, 5 % ignored                       seed 0
  C2  N=8192  D=4096 V=151936 bf16, 3 % ignored                       seed 0
  C3  C2 with a 4-bit affine group-64 head                             seed 0
  C4  B=1 Hq=32 Hkv=8 S in {8192; 2048, 4096, 16384} d=128 bf16 causal seed 0
  C5  16384 packed tokens (segments U[128, 4096], numpy rng 1), attention as C4 plus
      linear-CE at N=16384 with ignore_index at each segment's final token   seed 1
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

IGNORE_INDEX = -100


@dataclass
class CeInputs:
    hidden: torch.Tensor            # (N, D)
    weight: torch.Tensor | None     # (V, D) dense head
    w_q: torch.Tensor | None        # (V, D/8) int32 words
    scales: torch.Tensor | None     # (V, D/64)
    biases: torch.Tensor | None
    targets: torch.Tensor           # (N,) int64 with IGNORE_INDEX entries
    cotangent: torch.Tensor         # (N,) fp32: 1/num_valid on valid rows, 0 elsewhere
    num_valid: int


@dataclass
class AttnInputs:
    q: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor
    d_o: torch.Tensor
    scale: float
    seg_id: torch.Tensor | None = None
    seg_start: torch.Tensor | None = None
    seg_lengths: list | None = None


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def _targets(n: int, v: int, ignore_frac: float, g, device):
    t = torch.randint(0, v, (n,), generator=g, device=device, dtype=torch.int64)
    ign = torch.rand(n, generator=g, device=device) < ignore_frac
    t = torch.where(ign, torch.full_like(t, IGNORE_INDEX), t)
    return t


def _cotangent(t: torch.Tensor):
    valid = t != IGNORE_INDEX
    nv = int(valid.sum())
    return valid.to(torch.float32) / max(nv, 1), nv


def ce_dense(n: int, d: int, v: int, *, dtype=torch.bfloat16, ignore_frac: float = 0.03, seed: int = 0,
             device="cpu") -> CeInputs:
    """hidden ~ N(0,1); W ~ N(0, 1/sqrt(D)); targets uniform with `ignore_frac` masked."""
    g = _gen(seed, device)
    hidden = torch.randn(n, d, generator=g, device=device)
    w = torch.randn(v, d, generator=g, device=device) * (d ** -0.5)
    t = _targets(n, v, ignore_frac, g, device)
    ct, nv = _cotangent(t)
    return CeInputs(hidden.to(dtype), w.to(dtype), None, None, None, t, ct, nv)


def pack_int4_words(codes: torch.Tensor) -> torch.Tensor:
    """(V, D) codes in [0, 15] -> (V, D/8) int32 words, low nibble first
    (word[k >> 3] |= code << 4 * (k & 7))."""
    v, d = codes.shape
    c = codes.to(torch.int64).reshape(v, d // 8, 8)
    shifts = (4 * torch.arange(8, device=codes.device, dtype=torch.int64))[None, None, :]
    words = (c << shifts).sum(dim=-1)                      # < 2^32
    words = torch.where(words >= 2 ** 31, words - 2 ** 32, words)
    return words.to(torch.int32)


def ce_quant(n: int, d: int, v: int, *, ignore_frac: float = 0.03, seed: int = 0, device="cpu") -> CeInputs:
    """codes uniform in [0, 15]; scales = |N(0, 0.01)| (bf16); biases = -8 * scales; hidden bf16."""
    g = _gen(seed, device)
    codes = torch.randint(0, 16, (v, d), generator=g, device=device, dtype=torch.int64)
    scales = (torch.randn(v, d // 64, generator=g, device=device) * 0.01).abs().to(torch.bfloat16)
    biases = (-8.0 * scales.to(torch.float32)).to(torch.bfloat16)
    hidden = torch.randn(n, d, generator=g, device=device).to(torch.bfloat16)
    t = _targets(n, v, ignore_frac, g, device)
    ct, nv = _cotangent(t)
    return CeInputs(hidden, None, pack_int4_words(codes), scales, biases, t, ct, nv)


def attention(s: int, *, b: int = 1, hq: int = 32, hkv: int = 8, d: int = 128, dtype=torch.bfloat16, seed: int = 0,
              device="cpu") -> AttnInputs:
    g = _gen(seed, device)
    q = torch.randn(b, hq, s, d, generator=g, device=device).to(dtype)
    k = torch.randn(b, hkv, s, d, generator=g, device=device).to(dtype)
    v = torch.randn(b, hkv, s, d, generator=g, device=device).to(dtype)
    d_o = torch.randn(b, hq, s, d, generator=g, device=device).to(dtype)
    return AttnInputs(q, k, v, d_o, d ** -0.5)


def packed_lengths(total: int = 16384, lo: int = 128, hi: int = 4096, seed: int = 1) -> list:
    """Segment lengths drawn uniformly in [lo, hi] until `total` is filled; last one truncated."""
    rng = np.random.default_rng(seed)
    out, acc = [], 0
    while acc < total:
        n = int(rng.integers(lo, hi, endpoint=True))
        n = min(n, total - acc)
        out.append(n)
        acc += n
    return out


def segments_from_lengths(lengths, device="cpu"):
    ids = torch.repeat_interleave(torch.arange(len(lengths)), torch.tensor(lengths))
    starts = torch.repeat_interleave(torch.tensor([0] + list(np.cumsum(lengths)[:-1])), torch.tensor(lengths))
    return (ids.to(torch.int32)[None].contiguous().to(device), starts.to(torch.int32)[None].contiguous().to(device))


def packed(total: int = 16384, *, hq: int = 32, hkv: int = 8, d: int = 128, d_model: int = 4096, v: int = 151936,
           lo: int = 128, hi: int = 4096, seed: int = 1, device="cpu", with_ce: bool = True):
    """C5: packed attention inputs and the linear-CE inputs over the same tokens."""
    lengths = packed_lengths(total, lo, hi, seed)
    att = attention(total, hq=hq, hkv=hkv, d=d, seed=seed, device=device)
    att.seg_id, att.seg_start = segments_from_lengths(lengths, device)
    att.seg_lengths = lengths
    ce = None
    if with_ce:
        ce = ce_dense(total, d_model, v, ignore_frac=0.0, seed=seed, device=device)
        ends = torch.tensor(np.cumsum(lengths) - 1, device=ce.targets.device)
        ce.targets[ends] = IGNORE_INDEX
        ce.cotangent, ce.num_valid = _cotangent(ce.targets)
    return att, ce


# Algorithmic work (flops) of the two paths, used for TFLOP/s and roofline figures.
def ce_flops(n: int, d: int, v: int) -> float:
    """Three N x V x D contractions (logits, logit recompute, dH = G W): 6 N V D."""
    return 6.0 * n * v * d


def attn_flops(b: int, hq: int, s: int, d: int, seg_lengths=None) -> float:
    """Causal forward 2 GEMMs + backward 5 GEMMs at half the square: 7 B Hq S^2 d."""
    if seg_lengths is None:
        return 7.0 * b * hq * float(s) * s * d
    return 7.0 * b * hq * d * float(sum(float(x) * x for x in seg_lengths))
