"""Regenerate tests/golden/packing.json and tests/golden/planner.json from the REFERENCE's own
host-side code (read-only import from a checkout of IonDen/mlx-train-perf).

The reference's packer and planner are pure Python apart from `import mlx.core`; a permissive
stub for the `mlx` modules lets them import without MLX.  Nothing numeric on the two hot paths
can be produced this way (every such function touches an `mx.array`).

    python tests/golden/make_host_golden.py /path/to/mlx-train-perf
"""
import dataclasses
import json
import random
import sys
import types
from pathlib import Path

HERE = Path(__file__).resolve().parent


class _Anything(types.ModuleType):
    def __getattr__(self, name):
        if name.startswith("__"):
            raise AttributeError(name)
        return _Anything(f"{self.__name__}.{name}")

    def __call__(self, *a, **k):
        return _Anything("mlx.call")

    def __or__(self, other):      # `mx.array | None` in annotations evaluated at import time
        return self

    __ror__ = __or__

    def __mro_entries__(self, bases):   # `class X(nn.Module)` in the reference
        return (object,)


def _stub_mlx():
    for name in ("mlx", "mlx.core", "mlx.nn", "mlx.utils", "mlx.optimizers"):
        sys.modules[name] = _Anything(name)
    sys.modules["mlx"].core = sys.modules["mlx.core"]
    sys.modules["mlx"].nn = sys.modules["mlx.nn"]


def main(ref_root: str) -> None:
    _stub_mlx()
    sys.path.insert(0, str(Path(ref_root) / "src"))
    from mlx_train_perf.data import packing as rp
    from mlx_train_perf.plan import estimate as re_
    from mlx_train_perf.plan.calibration import load_calibration

    # ---------------------------------------------------------------- packer
    cases = []
    rng = random.Random(20261125)
    for case_id, (count, lo, hi, pack_len) in enumerate(
            [(40, 1, 30, 32), (200, 5, 900, 1024), (64, 1, 5, 4), (300, 100, 5000, 4096), (17, 1, 1, 1),
             (120, 1, 2100, 2048)]):
        lengths = [rng.randint(lo, hi) for _ in range(count)]
        for seed, epoch in ((0, 0), (7, 3)):
            packs = rp.pack_indices(lengths, pack_len, seed=seed, epoch=epoch)
            st = rp.pack_stats(packs, lengths, pack_len)
            cases.append({"kind": "pack", "lengths": lengths, "pack_len": pack_len, "seed": seed, "epoch": epoch,
                          "packs": packs, "stats": dataclasses.asdict(st)})
        bs = 2
        cases.append({"kind": "batching", "lengths": lengths, "pack_len": pack_len, "batch_size": bs,
                      "stock": dataclasses.asdict(rp.stock_batching_stats(lengths, batch_size=bs,
                                                                          max_seq_length=pack_len)),
                      "packed": dataclasses.asdict(rp.packed_batching_stats(lengths, pack_len, batch_size=bs,
                                                                            seed=1)),
                      "hist": dataclasses.asdict(rp.length_histogram(lengths))})
    rows = []
    for pack_len, spec in ((16, [(5, 0), (3, 2), (4, 9)]), (12, [(6, 0), (5, 1)]), (8, [(8, 3)]), (8, [(3, 0)]),
                           (10, [(1, 0), (1, 0), (1, 1), (2, 0)]), (9, [(4, 0), (4, 0)])):
        entries = [([rng.randint(1, 999) for _ in range(n)], off) for n, off in spec]
        row, sid, sst, mask = rp.build_row(entries, pack_len)
        rows.append({"pack_len": pack_len, "entries": entries, "row": row, "seg_id": sid, "seg_start": sst,
                     "loss_mask": mask})
    (HERE / "packing.json").write_text(json.dumps({"cases": cases, "rows": rows}))

    # ---------------------------------------------------------------- planner
    calib = load_calibration()
    shapes = {
        "qwen3_8b_4bit": dict(vocab=151936, hidden=4096, layers=36, intermediate=12288, heads=32, kv_heads=8,
                              tied=False, quant_bits=4, quant_group=64),
        "llama32_3b": dict(vocab=128256, hidden=3072, layers=28, intermediate=8192, heads=24, kv_heads=8,
                           tied=True, quant_bits=None, quant_group=None),
    }
    out = {"calibration": {f.name: getattr(calib, f.name) for f in dataclasses.fields(calib)}, "points": []}
    for sname, skw in shapes.items():
        shape = re_.ModelShape(**skw)
        for cfg_kw in (
            dict(batch=1, seq_len=8192, dtype="bfloat16", lora_rank=8, lora_layers=16, grad_checkpoint=True,
                 impl="kernel", attention="flash"),
            dict(batch=4, seq_len=2048, dtype="bfloat16", lora_rank=8, lora_layers=16, grad_checkpoint=True,
                 impl="naive", attention="stock"),
            dict(batch=2, seq_len=4096, dtype="float32", lora_rank=0, lora_layers=0, grad_checkpoint=False,
                 impl="chunked", attention="stock"),
        ):
            cfg = re_.TrainConfig(**cfg_kw)
            peak, comps = re_.estimate_peak(shape, cfg, calib)
            rep = re_.plan_fit(shape, cfg, budget_bytes=24 * 1024 ** 3)
            out["points"].append({"shape_name": sname, "shape": skw, "param_count": shape.param_count(),
                                  "cfg": cfg_kw, "peak": peak, "components": comps, "fits_24g": rep.fits,
                                  "suggestion": dataclasses.asdict(rep.suggestion) if rep.suggestion else None})
    # OLS refit: synthetic measurements generated from known coefficients must be recovered
    shape = re_.ModelShape(**shapes["qwen3_8b_4bit"])
    pts = []
    for seq in (1024, 2048, 4096, 8192):
        cfg = re_.TrainConfig(batch=1, seq_len=seq, dtype="bfloat16", lora_rank=8, lora_layers=16,
                              grad_checkpoint=True, impl="kernel", attention="stock")
        peak, comps = re_.estimate_peak(shape, cfg, calib)
        marginal = sum(v for k, v in comps.items() if k != "weights")
        pts.append({"cfg": dataclasses.asdict(cfg), "marginal": float(marginal)})
    fit = re_.fit_memory_coeffs(
        [re_.FitPoint(shape=shape, cfg=re_.TrainConfig(**p["cfg"]), marginal_peak_bytes=p["marginal"]) for p in pts],
        calib=calib)
    out["refit"] = {"shape": shapes["qwen3_8b_4bit"], "points": pts, "coeffs": fit}
    (HERE / "planner.json").write_text(json.dumps(out))
    print("wrote", HERE / "packing.json", HERE / "planner.json")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_host_golden.py /path/to/mlx-train-perf")
    main(sys.argv[1])
