"""Planner arithmetic against values computed by the reference's own `estimate_peak`,
`param_count`, `plan_fit` and `fit_memory_coeffs` (tests/golden/planner.json, written by
tests/golden/make_host_golden.py with the reference's published calibration), plus the HBM
retarget."""
import json
from pathlib import Path

import pytest

from mlx_train_perf_b200.errors import PlanInputError
from mlx_train_perf_b200.plan import estimate as E
from mlx_train_perf_b200.plan.calibration import load_calibration

GOLD = json.loads((Path(__file__).parent / "golden" / "planner.json").read_text())


def test_reference_calibration_file_matches_reference():
    c = load_calibration("reference")
    for k, v in GOLD["calibration"].items():
        if k != "provenance":
            assert getattr(c, k) == v
    assert c.kernel_loss_chunk_rows == 0


def test_peak_components_and_suggestions_match_reference():
    calib = load_calibration("reference")
    assert len(GOLD["points"]) == 6
    for p in GOLD["points"]:
        shape = E.ModelShape(**p["shape"])
        assert shape.param_count() == p["param_count"]
        cfg = E.TrainConfig(**p["cfg"])
        peak, comps = E.estimate_peak(shape, cfg, calib)
        assert comps == p["components"]
        assert peak == p["peak"]
        rep = E.plan_fit(shape, cfg, budget_bytes=24 * 1024 ** 3, calibration=calib)
        assert rep.fits == p["fits_24g"]
        got = None if rep.suggestion is None else {k: getattr(rep.suggestion, k) for k in p["suggestion"]}
        assert got == p["suggestion"]
        assert rep.headroom_bytes == rep.budget_bytes - rep.predicted_peak_bytes and rep.is_estimate


def test_refit_recovers_reference_coefficients():
    calib = load_calibration("reference")
    shape = E.ModelShape(**GOLD["refit"]["shape"])
    pts = [E.FitPoint(shape=shape, cfg=E.TrainConfig(**p["cfg"]), marginal_peak_bytes=p["marginal"])
           for p in GOLD["refit"]["points"]]
    got = E.fit_memory_coeffs(pts, calib=calib)
    for k, v in GOLD["refit"]["coeffs"].items():
        assert got[k] == pytest.approx(v, rel=1e-9)
    with pytest.raises(PlanInputError, match="rank-deficient"):
        E.fit_memory_coeffs(pts[:2], calib=calib)
    bad = E.FitPoint(shape=shape, cfg=E.TrainConfig(**{**GOLD["refit"]["points"][0]["cfg"], "impl": "naive"}),
                     marginal_peak_bytes=1.0)
    with pytest.raises(PlanInputError, match="impl='kernel'"):
        E.fit_memory_coeffs([bad], calib=calib)


def test_b200_retarget():
    calib = load_calibration()          # B200 default
    shape = E.ModelShape(vocab=151936, hidden=4096, layers=36, intermediate=12288, heads=32, kv_heads=8,
                         tied=False, quant_bits=4, quant_group=64)
    cfg = E.TrainConfig(batch=1, seq_len=8192, dtype="bfloat16", lora_rank=8, lora_layers=16,
                        grad_checkpoint=True, impl="kernel", attention="flash")
    peak, comps = E.estimate_peak(shape, cfg, calib)
    n = 8192
    # exact kernel workspace: ten balanced chunks of 15360 vocab rows (the bound is 16384 at this N), plus one
    # dequantised chunk of this 4-bit head
    assert E.kernel_loss_chunks(n, 151936, calib) == (15360, 10)
    assert E.kernel_loss_chunks(65536, 151936, calib) == (4096, 38)      # large N: the 512 MiB cap lowers the bound
    assert comps["loss"] == 3 * n * 4 + n * 15360 * 2 + n * 4096 * 4 + 15360 * 4096 * 2
    # O + L saved, plus the backward's transient per (head, token): the row statistics as a bf16 operand
    # tile (32 bytes) and the fp32 per-q-head dK / dV partials of a GQA model with head_dim 128
    # (2 * 128 * 4 bytes)
    assert calib.attn_bytes_per_head_token_flash == 1056.0
    assert comps["attention"] == n * 4096 * 2 + 32 * n * 4 + 1056 * 32 * n
    assert "max_memory_allocated" in calib.provenance["fit_source"] and len(calib.provenance["points"]) >= 8
    rep = E.plan_fit(shape, cfg)
    assert rep.fits and rep.budget_bytes > 150 * 1024 ** 3                 # one B200's HBM
    naive = E.estimate_peak(shape, E.TrainConfig(**{**cfg.__dict__, "impl": "naive"}), calib)[1]["loss"]
    assert naive > 100 * comps["loss"] / 10                                # (N, V) dwarfs the kernel workspace
    with pytest.raises(PlanInputError):
        E.estimate_peak(shape, E.TrainConfig(**{**cfg.__dict__, "dtype": "int8"}), calib)
    with pytest.raises(PlanInputError):
        E.estimate_peak(shape, E.TrainConfig(**{**cfg.__dict__, "attention": "ring"}), calib)
    with pytest.raises(PlanInputError):
        E.estimate_peak(shape, E.TrainConfig(**{**cfg.__dict__, "impl": "metal"}), calib)
    cfgd = E.ModelShape.from_config({"vocab_size": 10, "hidden_size": 8, "num_hidden_layers": 2,
                                     "intermediate_size": 16, "num_attention_heads": 4,
                                     "quantization": {"bits": 4, "group_size": 64}})
    assert cfgd.kv_heads == 4 and cfgd.tied is False and cfgd.quant_bits == 4


def test_kernel_loss_chunks_follow_the_library():
    """The planner's model of the fused loss backward's scratch is the library's own answer (the built
    library is asked for its workspace size; no GPU is needed for that)."""
    import ctypes as C
    from mlx_train_perf_b200 import _lib
    lib = _lib.load()
    calib = load_calibration()
    for n, d, v in ((8192, 4096, 151936), (16384, 4096, 151936), (512, 2048, 32000), (100000, 1024, 50000),
                    (8192, 4096, 18992), (300, 256, 40000)):
        a = _lib.CeArgs()
        a.hidden = a.weight = a.targets = 1 << 20        # placeholders; nothing is dereferenced
        a.n, a.d, a.v_local, a.dtype, a.impl = n, d, v, _lib.BF16, 0
        rows, count = E.kernel_loss_chunks(n, v, calib)
        want = n * rows * 2 + (n * d * 4 if count > 1 else 0)
        got = lib.b200tp_linear_ce_bwd_workspace_bytes(C.byref(a), _lib.BF16)
        assert want <= got <= want + 1024, (n, d, v, rows, count, got)
        # a 4-bit head: plus one dequantised chunk (the backward is always chunk-wise)
        a.weight, a.w_q, a.scales, a.biases = None, 1 << 20, 1 << 20, 1 << 20
        a.quant_bits, a.group_size, a.qparam_dtype = 4, 64, _lib.BF16
        if d % 64 == 0:
            rows, count = E.kernel_loss_chunks(n, v, calib)
            want = n * rows * 2 + (n * d * 4 if count > 1 else 0) + rows * d * 2
            got = lib.b200tp_linear_ce_bwd_workspace_bytes(C.byref(a), _lib.BF16)
            assert want <= got <= want + 1024, ("quant", n, d, v, rows, count, got)
