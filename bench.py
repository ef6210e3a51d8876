#!/usr/bin/env python
"""Benchmark of the two hot paths on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline (`metric` / `value`): fused linear-cross-entropy forward+backward tokens/s at
N=8192, D=4096, V=151936, bf16 (3 % of rows ignore_index), d_hidden with fp32 accumulation.
A "step" is one forward + one backward over that batch with the inputs already resident in
HBM.  At N GPUs the lm_head is vocab-sharded V/N per rank (strong scaling: the problem is
fixed): forward partial triples are all-gathered, the fp32 partial d_hidden is all-reduced,
both inside the timed region.  `e2e` is the same step through the public operator
(`linear_cross_entropy(...).backward()`) with the hidden states and targets copied from pinned
host memory every step (double-buffered: the copy for step i+1 is issued on a side stream while
step i computes) and the loss read back.

The `attention` object carries the second half of the metric: causal GQA flash attention
forward+backward TFLOP/s at S=8192, 32 q / 8 kv heads, d=128 (KV-head-group sharded at N>1,
no collective).

`--impl reference` times the CPU restatement of the reference's own chunked implementation
(the oracle; MLX itself cannot be installed here) on the host cores, rank 0 only.

One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

N_TOK, D_MODEL, VOCAB = 8192, 4096, 151936
ATT_S, ATT_HQ, ATT_HKV, ATT_D = 8192, 32, 8, 128
ATT_SETS = 72   # upper bound on the rotating attention input sets (enough of them are made to exceed L2)
CE_CHUNK_ROWS = 16384   # vocab rows per backward chunk inside the library

# dram__bytes_read.sum + dram__bytes_write.sum of one ce_logits_kernel<FWD> launch: captured
# with ncu at V=32768 (1.527e9 bytes, 128 vocab tiles; profiles/ce_kernels_v32768.md) and
# scaled by the vocab-tile count, which the traffic is proportional to.
CE_FWD_TRAFFIC_BYTES_PER_VTILE = 1.527e9 / 128


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"burst": float(d["bf16_tflops"]), "sustained": float(d["bf16_tflops_sustained"]),
                "hbm": float(d["hbm_gbs"]), "source": "measured"}
    return {"burst": 1590.0, "sustained": 1400.0, "hbm": 6650.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clock / throttle sampling during the timed region."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc = index, None
        self.t0 = self.t1 = None

    def launch(self):
        """Start nvidia-smi early (it takes a while to produce its first line)."""
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def start(self):
        if self.proc is None:
            self.launch()
        self.t0 = time.time()

    def stop(self) -> dict:
        self.t1 = time.time()
        time.sleep(0.12)
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        import datetime
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                if self.t0 is not None and not (self.t0 - 0.06 <= ts <= self.t1 + 0.06):
                    continue
            except ValueError:
                pass
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "power_w_max": max(power),
                "samples": len(sm), "reasons": sorted(reasons)}


def dist_setup(gpus: int):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"   # keep stdout to the one JSON line
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return world, rank, local


def timed_region(step, steps: int, warmup: int, world: int, device, sampler=None):
    """W untimed steps, then exactly K steps between barrier+synchronize pairs; device time by
    CUDA events on the launching stream; MAX over ranks."""
    import torch.distributed as dist
    for _ in range(warmup):
        step()
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(device)
    if sampler:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize(device)
    clocks = sampler.stop() if sampler else None
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(device)
    ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms.item()) / steps, clocks


def cpu_baseline_ce(w_cpu_f32, hidden_cpu_f32, targets_cpu, cotangent_cpu, budget_s: float = 15.0):
    """The oracle (a port of the reference's chunked path) on the host cores, on the first R
    rows of the same workload with the full vocabulary; R sized for about `budget_s` seconds."""
    from oracle import linear_ce as oc
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)

    def run(rows):
        t0 = time.perf_counter()
        _, lse, _ = oc.streamed_lse_and_target(hidden_cpu_f32[:rows], w_cpu_f32, targets_cpu[:rows])
        oc.chunked_backward(hidden_cpu_f32[:rows], w_cpu_f32, targets_cpu[:rows], lse, cotangent_cpu[:rows])
        return time.perf_counter() - t0

    probe = run(32)
    rows = int(max(32, min(2048, 32 * budget_s / max(probe, 1e-3))))
    rows = max(32, rows // 32 * 32)
    t = run(rows)
    return {"value": rows / t, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"first {rows} of {N_TOK} rows, full V={VOCAB}, fp32 torch-CPU, fwd+bwd, {t:.1f} s"}


def prestep_bandwidth(device, pk, steps):
    """The attention pre-step (per-head RMSNorm + RoPE on the q projection of the attention
    workload, batch 4 so a launch moves ~0.5 GB): HBM roofline of its forward kernel."""
    from mlx_train_perf_b200.attention.prestep import qk_norm_rope
    b, length, h, d = 4, ATT_S, ATT_HQ, ATT_D
    inv = 1.0 / (10000.0 ** (torch.arange(0, d, 2, dtype=torch.float32, device=device) / d))
    ang = torch.arange(length, dtype=torch.float32, device=device)[:, None] * inv[None]
    emb = torch.cat((ang, ang), -1)
    cos, sin = emb.cos().to(torch.bfloat16)[None].contiguous(), emb.sin().to(torch.bfloat16)[None].contiguous()
    xs = [torch.randn(b, length, h, d, device=device, dtype=torch.bfloat16) for _ in range(3)]   # > L2 together
    w = torch.ones(d, device=device, dtype=torch.bfloat16)
    n = max(10, steps * 2)
    with torch.no_grad():
        for i in range(5):
            qk_norm_rope(xs[i % 3], cos, sin, weight=w)
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n):
            qk_norm_rope(xs[i % 3], cos, sin, weight=w)
        e1.record()
        torch.cuda.synchronize(device)
    ms = e0.elapsed_time(e1) / n
    nbytes = 2 * xs[0].numel() * 2     # read + write, bf16
    gbs = nbytes / (ms / 1e3) / 1e9
    return {"kernel": "norm_rope_fwd_kernel", "shape": [b, length, h, d], "launch_us": ms * 1e3,
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": pk["hbm"], "unit": "GB/s", "frac": gbs / pk["hbm"],
                         "traffic": 285.0e6 + 223.5e6 if (length, h) == (8192, 32) else None},
            "gpu_launches": n}


def run_reference(args):
    """Reference arm: the CPU restatement of the reference's chunked forward + backward on the
    host cores, one bounded sample (rows of the same workload) per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from mlx_train_perf_b200 import configs
    from oracle import linear_ce as oc
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    rows = 1024   # large enough for the host BLAS to run at its rate; (steps + warm-up) x ~2-5 s in all
    inp = configs.ce_dense(rows, D_MODEL, VOCAB, dtype=torch.bfloat16, ignore_frac=0.03, seed=0)
    h, w = inp.hidden.float(), inp.weight.float()

    def step():
        _, lse, _ = oc.streamed_lse_and_target(h, w, inp.targets)
        oc.chunked_backward(h, w, inp.targets, lse, inp.cotangent)

    for _ in range(max(1, min(args.warmup, 2))):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    val = rows / dt
    line = {
        "impl": "reference", "metric": "linear_ce_fwd_bwd_tokens_per_s", "value": val, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"C2 fused linear-CE fwd+bwd(d_hidden) N={N_TOK} D={D_MODEL} V={VOCAB} bf16, "
                               "3% ignore_index, fp32 accumulation",
                   "parallelism": "host CPU", "sample_rows_per_step": rows},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": f"{rows} rows of the workload per step, full V, fp32 torch-CPU port of the "
                                   "reference's chunked forward+backward (MLX is not installable here)"},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


_REAL_STDOUT = None


def claim_stdout():
    """Keep stdout for the one JSON line: everything else this process or its libraries print there
    (NCCL's version banner, for one) is sent to stderr from here on."""
    global _REAL_STDOUT
    if _REAL_STDOUT is None:
        sys.stdout.flush()
        _REAL_STDOUT = os.dup(1)
        os.dup2(2, 1)


def emit(line: dict) -> None:
    data = (json.dumps(line) + "\n").encode()
    if _REAL_STDOUT is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        sys.stdout.flush()
        os.write(_REAL_STDOUT, data)


def main():
    claim_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-attention", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--small", action="store_true",
                    help="profiling case: V=32768 and S=4096 (inputs still exceed L2), no e2e / CPU legs")
    args = ap.parse_args()
    global VOCAB, ATT_S
    if args.small:
        VOCAB, ATT_S = 32768, 4096
        args.no_cpu_baseline = True
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
        return

    from mlx_train_perf_b200 import configs, parallel
    from mlx_train_perf_b200.attention import api as A
    from mlx_train_perf_b200.build import build
    from mlx_train_perf_b200.core import loss as L
    from mlx_train_perf_b200.core.loss import DenseHead, linear_cross_entropy

    world, rank, local = dist_setup(args.gpus)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path for the kernels)")
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if rank == 0:
        build(verbose=False)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    pk = peaks()

    # ------------------------------------------------------------------ linear-CE workload
    g = torch.Generator(device=device)
    g.manual_seed(0)
    hidden = torch.randn(N_TOK, D_MODEL, generator=g, device=device).to(torch.bfloat16)
    targets = torch.randint(0, VOCAB, (N_TOK,), generator=g, device=device, dtype=torch.int64)
    ign = torch.rand(N_TOK, generator=g, device=device) < 0.03
    targets = torch.where(ign, torch.full_like(targets, configs.IGNORE_INDEX), targets)
    valid = targets != configs.IGNORE_INDEX
    cotangent = valid.float() / valid.sum().clamp_min(1)
    lo, hi = parallel.shard_bounds(VOCAB, world, rank)
    gw = torch.Generator(device=device)
    gw.manual_seed(1000 + rank)
    weight = (torch.randn(hi - lo, D_MODEL, generator=gw, device=device) * D_MODEL ** -0.5).to(torch.bfloat16)
    head = DenseHead(weight=weight)
    v_local = hi - lo

    fwd_ms = []

    if world == 1:
        def step():
            f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            f0.record()
            _, _, _, lse, _ = L.ce_forward_raw(hidden, head, targets)
            f1.record()
            L.ce_backward_raw(hidden, head, targets, lse, cotangent)
            fwd_ms.append((f0, f1))
    else:
        sharded = parallel.VocabShardedLinearCE(head, lo)

        def step():
            f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            f0.record()
            _, lse, _ = sharded.forward(hidden, targets)
            f1.record()
            sharded.backward(hidden, targets, lse, cotangent)
            fwd_ms.append((f0, f1))

    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.launch()
    for _ in range(1):
        step()   # first call: module load, function attributes
    fwd_ms.clear()
    ms_step, clocks = timed_region(step, args.steps, args.warmup, world, device, sampler)
    L.check_device_status()
    timed = fwd_ms[-args.steps:]
    fwd_avg_ms = sum(a.elapsed_time(b) for a, b in timed) / len(timed)
    tokens_per_s = N_TOK / (ms_step / 1e3)
    chunks = -(-v_local // CE_CHUNK_ROWS)
    launches_per_step = 2 + 2 * chunks    # logits fwd + combine; (g, dH) per backward chunk
    fwd_flops = 2.0 * N_TOK * v_local * D_MODEL
    fwd_tflops = fwd_flops / (fwd_avg_ms / 1e3) / 1e12
    step_tflops = configs.ce_flops(N_TOK, D_MODEL, VOCAB) / (ms_step / 1e3) / 1e12 / world

    # ------------------------------------------------------------------ e2e through the public API
    hidden_host = hidden.cpu().pin_memory()
    targets_host = targets.cpu().pin_memory()

    # Double-buffered input pipeline, as a training loop's data loader would run it: step i+1's
    # host->device copies are issued on a side stream while step i's kernels run; every step still
    # copies its own inputs from pinned memory inside the timed region and reads its loss back.
    copy_stream = torch.cuda.Stream(device=device)
    pending = {}

    def prefetch(src_hidden):
        with torch.cuda.stream(copy_stream):
            h = src_hidden.to(device, non_blocking=True)
            t = targets_host.to(device, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(copy_stream)
        return h, t, ev

    def next_inputs(src_hidden):
        if "next" not in pending:
            pending["next"] = prefetch(src_hidden)
        h, t, ev = pending["next"]
        main = torch.cuda.current_stream(device)
        main.wait_event(ev)
        h.record_stream(main)
        t.record_stream(main)
        pending["next"] = prefetch(src_hidden)
        return h, t

    if world == 1:
        def e2e_step():
            h, t = next_inputs(hidden_host)
            h.requires_grad_(True)
            loss = linear_cross_entropy(h, head, t, reduction="mean", validate_targets=False)
            loss.backward()
            return float(loss.item())
    else:
        import torch.distributed as dist
        rows = N_TOK // world
        h_slice_host = hidden_host[rank * rows:(rank + 1) * rows].clone().pin_memory()

        def e2e_step():
            # every rank needs all rows (the vocabulary, not the batch, is sharded): copy 1/R of them
            # over PCIe and rebuild the batch over NVLink
            part, t = next_inputs(h_slice_host)
            h = torch.empty((N_TOK, D_MODEL), dtype=part.dtype, device=device)
            dist.all_gather_into_tensor(h, part)
            nll, lse, _ = sharded.forward(h, t)
            ct = (t != configs.IGNORE_INDEX).float()
            ct = ct / ct.sum().clamp_min(1)
            sharded.backward(h, t, lse, ct)
            return float((nll * ct).sum().item())

    e2e = None
    if not args.small:
        e2e_ms, _ = timed_region(e2e_step, args.steps, args.warmup, world, device)
        L.check_device_status()
        e2e = {"value": N_TOK / (e2e_ms / 1e3), "unit": "tokens/s",
               "h2d_bytes_per_step": hidden_host.numel() * 2 // world + targets_host.numel() * 8,
               "d2h_bytes_per_step": 4}

    # ------------------------------------------------------------------ CPU baseline (rank 0, N=1)
    cpu = None
    if world == 1 and rank == 0 and not args.no_cpu_baseline:
        cpu = cpu_baseline_ce(weight.float().cpu(), hidden_host.float(), targets_host, cotangent.cpu())

    # ------------------------------------------------------------------ attention workload
    att = None
    if not args.no_attention:
        del weight, head
        torch.cuda.empty_cache()
        # rotating input sets larger than L2 together, so no step finds its inputs cached
        att_sets = []
        set_bytes = 0
        for seed in range(ATT_SETS):
            inp = configs.attention(ATT_S, hq=ATT_HQ, hkv=ATT_HKV, d=ATT_D, seed=seed, device=device)
            q, k, v = parallel.shard_heads(inp.q, inp.k, inp.v, world, rank) if world > 1 else (inp.q, inp.k, inp.v)
            d_o = inp.d_o[:, parallel.head_shard(ATT_HKV, ATT_HQ, world, rank)[1]] if world > 1 else inp.d_o
            att_sets.append(tuple(x.contiguous() for x in (q, k, v, d_o)))
            set_bytes = sum(x.numel() * x.element_size() for x in att_sets[-1])
            if (seed + 1) * set_bytes > 160e6 and seed >= 1:
                break
        att_fwd = []
        att_calls = [0]

        def att_step():
            q, k, v, d_o = att_sets[att_calls[0] % len(att_sets)]
            att_calls[0] += 1
            f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            f0.record()
            o, lse = A.flash_fwd_raw(q, k, v, scale=inp.scale)
            f1.record()
            A.flash_bwd_raw(q, k, v, o, lse, d_o, scale=inp.scale)
            att_fwd.append((f0, f1))

        att_step()
        att_fwd.clear()
        att_sampler = ClockSampler(local) if rank == 0 else None
        if att_sampler:
            att_sampler.launch()
        # a step is ~4 ms: run 10x the steps so the region is long enough to sample clocks in
        att_steps = args.steps * 10
        att_ms, att_clocks = timed_region(att_step, att_steps, max(args.warmup, 10), world, device, att_sampler)
        L.check_device_status()
        # forward, row statistics, dQ, dK/dV; + the GQA reduce when dK/dV CTAs are per q head (small grids);
        # + the combine pass when the forward is split over keys
        fwd_split = A.flash_fwd_workspace_bytes(*att_sets[0][:3], scale=inp.scale) > 0
        q0_, k0_, v0_ = att_sets[0][:3]
        row_vec = q0_.shape[0] * q0_.shape[1] * q0_.shape[2] * 4
        dkv_partials = A.flash_bwd_workspace_bytes(q0_, k0_, v0_, scale=inp.scale) > 4 * row_vec   # else no reduce pass
        att_launches = 4 + int(fwd_split) + int(dkv_partials)
        tfl = configs.attn_flops(1, ATT_HQ, ATT_S, ATT_D) / (att_ms / 1e3) / 1e12
        a_fwd_ms = sum(a.elapsed_time(b) for a, b in att_fwd[-att_steps:]) / att_steps
        fwd_tfl = 2.0 * (ATT_HQ // world) * ATT_S * ATT_S * ATT_D / (a_fwd_ms / 1e3) / 1e12
        att = {"metric": "flash_attn_fwd_bwd_tflops", "value": tfl, "unit": "TFLOP/s", "ms_per_step": att_ms,
               "fwd_ms": a_fwd_ms, "config": {"workload": f"C4 causal GQA B=1 Hq={ATT_HQ} Hkv={ATT_HKV} S={ATT_S} d={ATT_D} bf16",
                                              "parallelism": f"kv-head-group x{world}",
                                              "l2": "%d rotating input sets, %.0f MB together (L2 is 126 MB)"
                                                    % (len(att_sets), len(att_sets) * set_bytes / 1e6)},
               "flops_model": "7*B*Hq*S^2*d",
               "roofline": {"bound": "tensor", "achieved": fwd_tfl, "peak": pk["sustained"], "unit": "TFLOP/s",
                            "frac": fwd_tfl / pk["sustained"], "traffic": None,
                            "kernel": "flash_fwd2_kernel" + (" (key range split) + flash_fwd_combine_kernel" if fwd_split else ""),
                            "peak_source": pk["source"] + " sustained"},
               "steps": att_steps, "clocks": att_clocks, "gpu_launches": att_launches * att_steps}
        if world == 1:
            att["prestep"] = prestep_bandwidth(device, pk, args.steps)

    if rank == 0:
        line = {
            "metric": "linear_ce_fwd_bwd_tokens_per_s", "value": tokens_per_s, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": f"C2 fused linear-CE fwd+bwd(d_hidden) N={N_TOK} D={D_MODEL} V={VOCAB} bf16, "
                                   "3% ignore_index, fp32 accumulation",
                       "parallelism": f"vocab-sharded x{world}" if world > 1 else "single GPU",
                       "l2": "inputs exceed L2 (lm_head shard %.2f GB vs 126 MB)" % (v_local * D_MODEL * 2 / 1e9)},
            "roofline": {"bound": "tensor", "achieved": fwd_tflops, "peak": pk["sustained"], "unit": "TFLOP/s",
                         "frac": fwd_tflops / pk["sustained"],
                         "traffic": CE_FWD_TRAFFIC_BYTES_PER_VTILE * (-(-v_local // 256)),
                         "kernel": "ce_logits_kernel<FWD> (+ the row combine kernel, a few microseconds)",
                         "launch_ms": fwd_avg_ms, "frac_of_burst": fwd_tflops / pk["burst"],
                         "peak_source": pk["source"] + " sustained (kernel timed inside a long step)"},
            "step_tflops_per_gpu": step_tflops, "step_frac_of_sustained": step_tflops / pk["sustained"],
            "flops_model": "6*N*V*D",
            "cpu_baseline": cpu,
            "e2e": e2e,
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
            "attention": att,
        }
        emit(line)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
