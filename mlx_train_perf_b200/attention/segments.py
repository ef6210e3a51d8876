"""Packed-sequence segment carrier (src/mlx_train_perf/attention/segments.py:8-29)."""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class PackedMask:
    """Block-diagonal-causal segment description of one packed batch.

    seg_id: int32 (B, L) -- ascending segment ids per position, starting at 0 in each row;
      gapless (the pad tail is the row's last segment).
    seg_start: int32 (B, L) -- index where the position's segment begins (non-decreasing).

    Key j is visible to query i iff seg_id[j] == seg_id[i] and j <= i.
    """
    seg_id: torch.Tensor
    seg_start: torch.Tensor


def segment_allowed(seg_id: torch.Tensor) -> torch.Tensor:
    """(B, 1, N, N) bool visibility mask; O(N^2), for tests and tiny inputs only."""
    same = seg_id[:, None, :, None] == seg_id[:, None, None, :]
    n = seg_id.shape[-1]
    causal = torch.tril(torch.ones(n, n, dtype=torch.bool, device=seg_id.device))[None, None]
    return same & causal
