"""Re-measure the fit planner's memory coefficients on the GPU at hand.

    python -m mlx_train_perf_b200.plan.measure [--out calibration_b200.json]

Builds a random-init Llama-shaped model (no checkpoint needed), freezes it, attaches rank-8 LoRA
adapters to q_proj / v_proj of every layer (the planner's adapter model: two modules, two
matrices), and runs AdamW train steps through the fused linear-cross-entropy loss at a grid of
sequence lengths with the stock (materialising) attention and with `enable_flash_attention`,
checkpointed and not.  Each point records the MARGINAL peak -- `torch.cuda.max_memory_allocated`
above what was resident when only the frozen weights were loaded -- and
`plan.estimate.fit_memory_coeffs` turns the points into the coefficients, as the reference's
campaign does on its machine (plan/estimate.py:350-491 of the reference).
"""
from __future__ import annotations

import argparse
import datetime
import json
from pathlib import Path

import torch
from torch import nn

from mlx_train_perf_b200.adapters.torch_lm import split_model
from mlx_train_perf_b200.attention.wrapper import enable_flash_attention
from mlx_train_perf_b200.core.loss import DenseHead, linear_cross_entropy
from mlx_train_perf_b200.plan import estimate as E
from mlx_train_perf_b200.plan.calibration import Calibration, load_calibration

_DIR = Path(__file__).resolve().parent


class LoRALinear(nn.Module):
    """y = W x + B (A x): frozen base, trainable rank-r factors (bf16 like the base)."""

    def __init__(self, base: nn.Linear, rank: int):
        super().__init__()
        self.base = base
        self.a = nn.Parameter(torch.randn(rank, base.in_features, dtype=base.weight.dtype,
                                          device=base.weight.device) * 0.01)
        self.b = nn.Parameter(torch.zeros(base.out_features, rank, dtype=base.weight.dtype,
                                          device=base.weight.device))

    def forward(self, x):
        return self.base(x) + (x @ self.a.t()) @ self.b.t()


def _model(cfg_kw: dict, device):
    import transformers
    torch.manual_seed(0)
    m = transformers.LlamaForCausalLM(transformers.LlamaConfig(**cfg_kw)).to(device=device, dtype=torch.bfloat16)
    for p in m.parameters():
        p.requires_grad_(False)
    return m


def _attach_lora(m, rank: int):
    params = []
    for layer in m.model.layers:
        att = layer.self_attn
        att.q_proj = LoRALinear(att.q_proj, rank)
        att.v_proj = LoRALinear(att.v_proj, rank)
        params += [att.q_proj.a, att.q_proj.b, att.v_proj.a, att.v_proj.b]
    return params


def measure_point(cfg_kw: dict, shape: E.ModelShape, cfg: E.TrainConfig, device, steps: int = 3) -> float:
    """Marginal peak bytes of `steps` train steps at `cfg` (the frozen weights excluded)."""
    torch.cuda.synchronize(device)
    torch.cuda.empty_cache()
    before = torch.cuda.memory_allocated(device)
    m = _model(cfg_kw, device)
    m.config._attn_implementation = "eager"
    torch.cuda.synchronize(device)
    resident = torch.cuda.memory_allocated(device)          # the frozen weights (+ what was there before)
    params = _attach_lora(m, cfg.lora_rank)
    if cfg.attention == "flash":
        enable_flash_attention(m)
    if cfg.grad_checkpoint:
        m.gradient_checkpointing_enable(gradient_checkpointing_kwargs={"use_reentrant": False})
    m.train()
    opt = torch.optim.AdamW(params, lr=1e-4)
    head = DenseHead(weight=m.lm_head.weight, trainable=False)
    if cfg.attention == "flash":
        trunk, _ = split_model(m)                                        # walks the wrapped layers, causal mask
    else:
        trunk = lambda ids: m.model(input_ids=ids, use_cache=False).last_hidden_state
    g = torch.Generator(device=device).manual_seed(1)
    batch = torch.randint(1, shape.vocab, (cfg.batch, cfg.seq_len + 1), generator=g, device=device)
    torch.cuda.reset_peak_memory_stats(device)
    for _ in range(steps):
        hidden = trunk(batch[:, :-1])                                    # trunk only: no (N, V) logits
        loss = linear_cross_entropy(hidden, head, batch[:, 1:], validate_targets=False)
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
    torch.cuda.synchronize(device)
    peak = torch.cuda.max_memory_allocated(device) - resident
    del m, opt, params, loss, hidden, head, batch, trunk
    torch.cuda.empty_cache()
    assert torch.cuda.memory_allocated(device) <= before + (64 << 20), "a measurement point leaked device memory"
    return float(peak)


def run(device, *, verbose: bool = True):
    cfg_kw = dict(vocab_size=32000, hidden_size=2048, intermediate_size=5632, num_hidden_layers=8,
                  num_attention_heads=16, num_key_value_heads=4, max_position_embeddings=16384,
                  attention_dropout=0.0, tie_word_embeddings=False)
    shape = E.ModelShape.from_config(cfg_kw)
    mk = lambda s, gc, att: E.TrainConfig(batch=1, seq_len=s, dtype="bfloat16", lora_rank=8, lora_layers=8,
                                          grad_checkpoint=gc, impl="kernel", attention=att)
    grid = ([mk(s, True, "stock") for s in (1024, 2048, 3072, 4096)] + [mk(s, False, "stock") for s in (1024, 2048)]
            + [mk(s, False, "flash") for s in (2048, 4096, 8192)] + [mk(4096, True, "flash")])
    points = []
    for cfg in grid:
        peak = measure_point(cfg_kw, shape, cfg, device)
        points.append(E.FitPoint(shape=shape, cfg=cfg, marginal_peak_bytes=peak))
        if verbose:
            print(f"seq {cfg.seq_len:5d} gc {int(cfg.grad_checkpoint)} {cfg.attention:5s}: {peak / 2**20:9.1f} MiB", flush=True)
    return shape, points


def flash_transient_bytes_per_head_token(shape: E.ModelShape, seq_len: int = 4096) -> float:
    """Exact backward workspace of the flash kernels per (query head, token), asked of the library
    (the row statistics as a 32-byte bf16 tile row, plus the fp32 per-q-head dK / dV partials when heads share kv heads and the
    grid is small enough that each q head gets its own dK / dV CTAs; at the default 4096 tokens that
    holds for models of up to 7 kv heads, so the figure is an upper bound for larger ones)."""
    import ctypes as C

    from mlx_train_perf_b200 import _lib
    a = _lib.AttnArgs()
    a.b, a.hq, a.hkv, a.s, a.d = 1, shape.heads, shape.kv_heads, seq_len, shape.hidden // shape.heads
    a.dtype, a.causal, a.scale = _lib.BF16, 1, 1.0
    for arr, h in ((a.q_stride, a.hq), (a.k_stride, a.hkv), (a.v_stride, a.hkv), (a.o_stride, a.hq)):
        arr[0], arr[1], arr[2] = h * a.s * a.d, a.s * a.d, a.d
    return _lib.load().b200tp_flash_bwd_workspace_bytes(C.byref(a)) / float(shape.heads * seq_len)


def fit(points, shape: E.ModelShape, old: Calibration) -> dict:
    """Coefficients from the measured points.

    (base, quadratic) come from the reference's least-squares step on the checkpointed stock points
    (`fit_memory_coeffs`).  The flash transient is not fitted but taken exactly from the library's
    workspace size.  The two linear activation coefficients are then through-origin fits on the
    FLASH points (the path this planner recommends), checkpointed and not: the model has one linear
    coefficient per checkpointing mode, and the stock un-checkpointed path also keeps every layer's
    (S, S) probabilities, which that form cannot express -- such configurations are under-predicted
    and the provenance says so."""
    stock = [p for p in points if p.cfg.attention == "stock" and p.cfg.grad_checkpoint]
    s1 = E.fit_memory_coeffs(stock, calib=old)
    base, a_quad = s1["base_transient_bytes"], s1["attn_bytes_per_head_token2"]
    a_flash = flash_transient_bytes_per_head_token(shape)

    def lin(ps, fallback):
        num = den = 0.0
        for p in ps:
            x_lin = float(p.cfg.batch * p.cfg.seq_len * p.shape.hidden * p.shape.layers)
            fixed = (E._lora_bytes(p.cfg, p.shape) + E._optimizer_bytes(p.cfg, p.shape, old)
                     + E._loss_bytes(p.cfg, p.shape, old) + E._flash_saved_state_bytes(p.cfg, p.shape)
                     + a_flash * p.cfg.batch * p.shape.heads * p.cfg.seq_len + base)
            num += (p.marginal_peak_bytes - fixed) * x_lin
            den += x_lin * x_lin
        return max(0.0, num / den) if den else fallback

    flash = [p for p in points if p.cfg.attention == "flash"]
    a_full = lin([p for p in flash if not p.cfg.grad_checkpoint], old.act_bytes_per_token_hidden_layer_full)
    a_ckpt = max(lin([p for p in flash if p.cfg.grad_checkpoint], old.act_bytes_per_token_hidden_layer_ckpt),
                 s1["act_bytes_per_token_hidden_layer_ckpt"], 0.0)
    return {"base_transient_bytes": max(0.0, base), "act_bytes_per_token_hidden_layer_ckpt": a_ckpt,
            "act_bytes_per_token_hidden_layer_full": a_full, "attn_bytes_per_head_token2": a_quad,
            "attn_bytes_per_head_token_flash": a_flash}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=str(_DIR / "calibration_b200.json"))
    args = ap.parse_args()
    device = torch.device("cuda", 0)
    old = load_calibration("b200")
    shape, points = run(device)
    new = {**{k: v for k, v in old.__dict__.items() if k != "provenance"}, **fit(points, shape, old)}
    calib = Calibration(**{**new, "provenance": {}})

    def rel_err(p):
        pred = E.estimate_peak(p.shape, p.cfg, calib)[0] / (1 + calib.overhead_frac) - E._weights_bytes(p.shape, 2)
        return (pred - p.marginal_peak_bytes) / p.marginal_peak_bytes

    errs = [{"seq_len": p.cfg.seq_len, "grad_checkpoint": p.cfg.grad_checkpoint, "attention": p.cfg.attention,
             "marginal_peak_bytes": p.marginal_peak_bytes, "relative_error_of_fit": round(rel_err(p), 4)}
            for p in points]
    new["provenance"] = {
        "machine": torch.cuda.get_device_name(device),
        "cuda": torch.version.cuda, "torch": torch.__version__,
        "measured_date": datetime.date.today().isoformat(),
        "fit_source": "python -m mlx_train_perf_b200.plan.measure: torch.cuda.max_memory_allocated marginal peaks of "
                      "LoRA (rank 8, q_proj / v_proj) AdamW train steps of a random-init Llama-shaped model "
                      f"(hidden {shape.hidden}, {shape.layers} layers, {shape.heads}/{shape.kv_heads} heads, vocab "
                      f"{shape.vocab}) through the fused loss, stock (eager) and flash attention; base and the "
                      "quadratic coefficient by least squares on the checkpointed stock points, the flash transient "
                      "from the library's exact workspace size, the linear coefficients from the flash points "
                      "(stock un-checkpointed runs also keep every layer's (S, S) probabilities and are "
                      "under-predicted by this model form)",
        "points": errs,
    }
    Path(args.out).write_text(json.dumps(new, indent=2) + "\n")
    print(json.dumps({k: v for k, v in new.items() if k != "provenance"}, indent=2))
    for e in errs:
        print(e)


if __name__ == "__main__":
    main()
