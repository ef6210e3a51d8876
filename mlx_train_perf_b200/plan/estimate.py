"""Analytic memory-fit planner, retargeted from unified memory to one GPU's HBM
(src/mlx_train_perf/plan/estimate.py:57-135, :210-347 planner; :350-491 coefficient refit).

Peak = (weights + base + LoRA + AdamW + linear activations + attention + loss) x (1 + overhead).
Attention is either "stock" (a materialised (N, N) backward) or "flash" (saved O + L plus a
linear transient); the loss is "naive" (full logits), "chunked" (one 8192-column tile) or
"kernel" (no logits: three N-length fp32 vectors, plus -- with the B200 calibration -- the
backward's (N, chunk) bf16 tile and (N, D) fp32 accumulator).  Pure arithmetic; the only
device query is the default budget.
"""
from __future__ import annotations

from collections.abc import Iterator
from dataclasses import dataclass, replace
from typing import Any

from mlx_train_perf_b200.errors import PlanInputError
from mlx_train_perf_b200.plan.calibration import Calibration, load_calibration

DTYPE_BYTES = {"float32": 4, "bfloat16": 2, "float16": 2}
CHUNK_TILE = 8192          # the chunked loss impl's fixed vocab tile
LORA_MODULES = 2           # q_proj, v_proj
LORA_MATRICES = 2          # A, B
B200_HBM_BYTES = 183_359 * 1024 ** 2   # what nvidia-smi reports for one B200
BUDGET_FRACTION = 0.92     # default share of device memory the plan may use


@dataclass(frozen=True)
class ModelShape:
    vocab: int
    hidden: int
    layers: int
    intermediate: int
    heads: int
    kv_heads: int
    tied: bool
    quant_bits: int | None
    quant_group: int | None

    def param_count(self) -> int:
        """Llama / Qwen3 arithmetic: embedding V D (+ untied head V D); per layer attention
        2 D D (heads + kv) / heads, MLP 3 D I, two norms; final norm."""
        d = self.hidden
        per_layer = 2 * d * d * (self.heads + self.kv_heads) // self.heads + 3 * d * self.intermediate + 2 * d
        return self.vocab * d * (1 if self.tied else 2) + self.layers * per_layer + d

    @classmethod
    def from_config(cls, config: dict[str, Any]) -> "ModelShape":
        """From a HF `config.json` dict; an optional `quantization` block gives bits / group."""
        heads = int(config["num_attention_heads"])
        quant = config.get("quantization") or config.get("quantization_config")
        return cls(vocab=int(config["vocab_size"]), hidden=int(config["hidden_size"]),
                   layers=int(config["num_hidden_layers"]), intermediate=int(config["intermediate_size"]),
                   heads=heads, kv_heads=int(config.get("num_key_value_heads", heads)),
                   tied=bool(config.get("tie_word_embeddings", False)),
                   quant_bits=int(quant["bits"]) if quant and "bits" in quant else None,
                   quant_group=int(quant["group_size"]) if quant and "group_size" in quant else None)


@dataclass(frozen=True)
class TrainConfig:
    batch: int
    seq_len: int
    dtype: str
    lora_rank: int
    lora_layers: int
    grad_checkpoint: bool
    impl: str
    attention: str = "stock"


@dataclass(frozen=True)
class FitReport:
    fits: bool
    predicted_peak_bytes: int
    budget_bytes: int
    headroom_bytes: int
    components: dict
    suggestion: TrainConfig | None
    is_estimate: bool
    provenance: dict


@dataclass(frozen=True)
class FitPoint:
    """One measured train-step MARGINAL peak (bytes above what was resident before the loop)."""
    shape: ModelShape
    cfg: TrainConfig
    marginal_peak_bytes: float


def _dtype_bytes(dtype: str) -> int:
    if dtype not in DTYPE_BYTES:
        raise PlanInputError(f"unknown dtype {dtype!r}; expected one of {sorted(DTYPE_BYTES)}")
    return DTYPE_BYTES[dtype]


def _weights_bytes(shape: ModelShape, dtype_size: int) -> int:
    p = shape.param_count()
    if shape.quant_bits is None or shape.quant_group is None:
        return p * dtype_size
    return int(p * (shape.quant_bits / 8 + 4 / shape.quant_group))   # codes + bf16 scale and bias per group


def _lora_params(cfg: TrainConfig, shape: ModelShape) -> int:
    return cfg.lora_layers * LORA_MODULES * LORA_MATRICES * cfg.lora_rank * shape.hidden


def _lora_bytes(cfg: TrainConfig, shape: ModelShape) -> int:
    return 2 * _lora_params(cfg, shape)


def _optimizer_bytes(cfg: TrainConfig, shape: ModelShape, calib: Calibration) -> int:
    return int(calib.optimizer_bytes_per_param * _lora_params(cfg, shape))


def _activation_bytes(cfg: TrainConfig, shape: ModelShape, calib: Calibration) -> int:
    coef = (calib.act_bytes_per_token_hidden_layer_ckpt if cfg.grad_checkpoint
            else calib.act_bytes_per_token_hidden_layer_full)
    return int(coef * cfg.batch * cfg.seq_len * shape.hidden * shape.layers)


def _flash_saved_state_bytes(cfg: TrainConfig, shape: ModelShape) -> int:
    """O (batch x seq x hidden, compute dtype) + L (batch x heads x seq, fp32)."""
    return (cfg.batch * cfg.seq_len * shape.hidden * _dtype_bytes(cfg.dtype)
            + cfg.batch * shape.heads * cfg.seq_len * 4)


def _attention_bytes(cfg: TrainConfig, shape: ModelShape, calib: Calibration) -> int:
    if cfg.attention == "stock":
        return int(calib.attn_bytes_per_head_token2 * cfg.batch * shape.heads * cfg.seq_len ** 2)
    if cfg.attention == "flash":
        return int(_flash_saved_state_bytes(cfg, shape)
                   + calib.attn_bytes_per_head_token_flash * cfg.batch * shape.heads * cfg.seq_len)
    raise PlanInputError(f"unknown attention {cfg.attention!r}; expected 'stock' or 'flash'")


def kernel_loss_chunks(n: int, vocab: int, calib: Calibration) -> tuple[int, int]:
    """(rows per chunk, chunk count) of the fused loss backward, as the library picks them: the bound is
    `kernel_loss_chunk_rows`, lowered (not below 2048) so that the (N, chunk) bf16 tile fits
    `kernel_loss_scratch_bytes`; the vocabulary is spread evenly over the fewest chunks the bound allows,
    in multiples of 256 rows."""
    bound = calib.kernel_loss_chunk_rows
    if calib.kernel_loss_scratch_bytes > 0:
        fit = calib.kernel_loss_scratch_bytes // (2 * max(n, 1)) // 256 * 256
        bound = min(bound, max(2048, fit))
    count = -(-vocab // bound)
    rows = -(-(-(-vocab // count)) // 256) * 256
    return rows, count


def _loss_bytes(cfg: TrainConfig, shape: ModelShape, calib: Calibration) -> int:
    n = cfg.batch * cfg.seq_len
    if cfg.impl == "naive":
        base = int(calib.naive_loss_bytes_per_nv * n * shape.vocab)
    elif cfg.impl == "chunked":
        base = n * CHUNK_TILE * 4 * 3
    elif cfg.impl == "kernel":
        base = 3 * n * 4
        if calib.kernel_loss_chunk_rows > 0:
            quantized = bool(shape.quant_bits)
            rows, count = kernel_loss_chunks(n, shape.vocab, calib)
            base += n * rows * 2 + (n * shape.hidden * 4 if count > 1 else 0)   # g tile; fp32 accumulator over chunks
            if quantized and n > 512:
                base += rows * shape.hidden * 2                                   # one dequantised chunk of the head
    else:
        raise PlanInputError(f"unknown impl {cfg.impl!r}; expected 'naive', 'chunked', or 'kernel'")
    if cfg.lora_rank == 0:          # full fine-tuning: the head's fp32 gradient, doubled by the concat
        base += shape.vocab * shape.hidden * 4 * 2
    return base


def estimate_peak(shape: ModelShape, cfg: TrainConfig, calib: Calibration) -> tuple[int, dict]:
    """Predicted peak bytes and the component breakdown; no I/O, no device query."""
    components = {
        "weights": _weights_bytes(shape, _dtype_bytes(cfg.dtype)),
        "base": int(calib.base_transient_bytes),
        "lora": _lora_bytes(cfg, shape),
        "optimizer": _optimizer_bytes(cfg, shape, calib),
        "activations": _activation_bytes(cfg, shape, calib),
        "attention": _attention_bytes(cfg, shape, calib),
        "loss": _loss_bytes(cfg, shape, calib),
    }
    return int(sum(components.values()) * (1 + calib.overhead_frac)), components


def _candidates(cfg: TrainConfig) -> Iterator[TrainConfig]:
    """Halve the batch down to 1, then step seq_len down by 1024 to a floor of 1024."""
    b = cfg.batch
    while b > 1:
        b = max(1, b // 2)
        yield replace(cfg, batch=b)
    s = cfg.seq_len
    while s > 1024:
        s = max(1024, s - 1024)
        yield replace(cfg, batch=1, seq_len=s)


def default_budget_bytes() -> int:
    """0.92 of the current CUDA device's total memory, or of a nominal B200 when no device
    is visible (planning on a login node)."""
    try:
        import torch
        if torch.cuda.is_available():
            return int(BUDGET_FRACTION * torch.cuda.mem_get_info()[1])
    except Exception:   # pragma: no cover - planning must not need a GPU
        pass
    return int(BUDGET_FRACTION * B200_HBM_BYTES)


def plan_fit(shape: ModelShape, cfg: TrainConfig, *, budget_bytes: int | None = None,
             calibration: Calibration | None = None) -> FitReport:
    calib = calibration or load_calibration()
    budget = default_budget_bytes() if budget_bytes is None else budget_bytes
    peak, components = estimate_peak(shape, cfg, calib)
    fits = peak <= budget
    suggestion = None
    if not fits:
        suggestion = next((c for c in _candidates(cfg) if estimate_peak(shape, c, calib)[0] <= budget), None)
    return FitReport(fits=fits, predicted_peak_bytes=peak, budget_bytes=budget, headroom_bytes=budget - peak,
                     components=components, suggestion=suggestion, is_estimate=True, provenance=calib.provenance)


def fit_memory_coeffs(points: list[FitPoint], *, calib: Calibration) -> dict:
    """Refit the measured coefficients from kernel-impl train-step marginal peaks.

    marginal = base + a_lin[gc] x_lin + a_quad x_quad + analytic(lora + optimizer + loss), with
    x_lin = batch seq hidden layers, x_quad = batch heads seq^2.  Stock, checkpointed points give
    (base, a_lin_ckpt, a_quad) by least squares (the design must have rank 3, else
    PlanInputError -- least squares would silently return a minimum-norm answer); stock,
    un-checkpointed points then give a_lin_full alone.  Flash points give a_flash by a
    one-variable through-origin fit of the residual after base, a_lin (from `calib`) and the
    analytic saved state: x_flash = batch heads seq is collinear with x_lin at a fixed shape."""
    import numpy as np

    for p in points:
        if p.cfg.impl != "kernel":
            raise PlanInputError(f"fit_memory_coeffs only accepts impl='kernel' FitPoints (got impl={p.cfg.impl!r})")

    def resid(p):
        return p.marginal_peak_bytes - (_lora_bytes(p.cfg, p.shape) + _optimizer_bytes(p.cfg, p.shape, calib)
                                        + _loss_bytes(p.cfg, p.shape, calib))

    def x_lin(p):
        return float(p.cfg.batch * p.cfg.seq_len * p.shape.hidden * p.shape.layers)

    def x_quad(p):
        return float(p.cfg.batch * p.shape.heads * p.cfg.seq_len ** 2)

    def x_flash(p):
        return float(p.cfg.batch * p.shape.heads * p.cfg.seq_len)

    stock = [p for p in points if p.cfg.attention == "stock"]
    flash = [p for p in points if p.cfg.attention == "flash"]
    base, a_ckpt = float(calib.base_transient_bytes), calib.act_bytes_per_token_hidden_layer_ckpt
    a_full, a_quad = calib.act_bytes_per_token_hidden_layer_full, calib.attn_bytes_per_head_token2
    if stock:
        ck = [p for p in stock if p.cfg.grad_checkpoint]
        design = np.array([[1.0, x_lin(p), x_quad(p)] for p in ck], dtype=float).reshape(-1, 3)
        if np.linalg.matrix_rank(design) < 3:
            raise PlanInputError(
                "fit_memory_coeffs cannot separate (base, linear, quadratic): the gc=True design matrix is "
                f"rank-deficient ({len(ck)} gc=True stock point(s), {len({p.cfg.seq_len for p in ck})} distinct "
                "seq_len; with batch fixed at least 3 distinct seq_len are needed)")
        sol = np.linalg.lstsq(design, np.array([resid(p) for p in ck], dtype=float), rcond=None)[0]
        base, a_ckpt, a_quad = float(sol[0]), float(sol[1]), float(sol[2])
        nock = [p for p in stock if not p.cfg.grad_checkpoint]
        den = sum(x_lin(p) ** 2 for p in nock)
        if den:
            a_full = sum((resid(p) - base - a_quad * x_quad(p)) * x_lin(p) for p in nock) / den
    a_flash = calib.attn_bytes_per_head_token_flash
    if flash:
        den = sum(x_flash(p) ** 2 for p in flash)
        if den <= 0:
            raise PlanInputError("fit_memory_coeffs cannot identify a_flash: sum(x_flash^2) == 0")

        def fres(p):
            a = (calib.act_bytes_per_token_hidden_layer_ckpt if p.cfg.grad_checkpoint
                 else calib.act_bytes_per_token_hidden_layer_full)
            return resid(p) - calib.base_transient_bytes - a * x_lin(p) - _flash_saved_state_bytes(p.cfg, p.shape)

        a_flash = sum(fres(p) * x_flash(p) for p in flash) / den
    return {"base_transient_bytes": base, "act_bytes_per_token_hidden_layer_ckpt": a_ckpt,
            "act_bytes_per_token_hidden_layer_full": float(a_full), "attn_bytes_per_head_token2": a_quad,
            "attn_bytes_per_head_token_flash": float(a_flash)}
