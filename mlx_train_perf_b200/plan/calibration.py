"""Calibration constants of the fit planner (src/mlx_train_perf/plan/calibration.py:22-85).

Two versioned data files carry their own provenance:
  `calibration_b200.json`       -- default; HBM budget model for one B200 (180 GB HBM3e)
  `calibration_reference.json`  -- the reference's published M1 Max numbers, kept so the
                                   planner arithmetic can be checked against the reference's
                                   own outputs (tests/golden/planner.json)
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path

_DIR = Path(__file__).resolve().parent


@dataclass(frozen=True)
class Calibration:
    base_transient_bytes: float                    # fixed per-run runtime floor
    act_bytes_per_token_hidden_layer_ckpt: float   # linear activations, checkpointing on
    act_bytes_per_token_hidden_layer_full: float   # linear activations, checkpointing off
    attn_bytes_per_head_token2: float              # materialised attention backward, per head*seq^2
    attn_bytes_per_head_token_flash: float         # flash backward live transient, per head*seq
    optimizer_bytes_per_param: float               # AdamW: two fp32 moments
    overhead_frac: float
    naive_loss_bytes_per_nv: float
    provenance: dict
    # Vocab rows per backward chunk of the fused loss kernels: the kernel path holds one
    # (N, chunk) bf16 tile of g and an (N, D) fp32 accumulator.  0 = the reference's kernel
    # model (three N-length fp32 vectors only).
    kernel_loss_chunk_rows: int = 0
    # The library lowers that bound so that the (N, chunk) tile stays within this many bytes (0 = no cap).
    kernel_loss_scratch_bytes: int = 0


def load_calibration(name: str = "b200") -> Calibration:
    path = _DIR / f"calibration_{name}.json"
    if not path.exists():
        raise FileNotFoundError(f"no calibration file {path.name}; known: b200, reference")
    raw = json.loads(path.read_text())
    return Calibration(
        base_transient_bytes=float(raw["base_transient_bytes"]),
        act_bytes_per_token_hidden_layer_ckpt=float(raw["act_bytes_per_token_hidden_layer_ckpt"]),
        act_bytes_per_token_hidden_layer_full=float(raw["act_bytes_per_token_hidden_layer_full"]),
        attn_bytes_per_head_token2=float(raw["attn_bytes_per_head_token2"]),
        attn_bytes_per_head_token_flash=float(raw["attn_bytes_per_head_token_flash"]),
        optimizer_bytes_per_param=float(raw["optimizer_bytes_per_param"]),
        overhead_frac=float(raw["overhead_frac"]),
        naive_loss_bytes_per_nv=float(raw["naive_loss_bytes_per_nv"]),
        provenance=dict(raw["provenance"]),
        kernel_loss_chunk_rows=int(raw.get("kernel_loss_chunk_rows", 0)),
        kernel_loss_scratch_bytes=int(raw.get("kernel_loss_scratch_bytes", 0)),
    )
