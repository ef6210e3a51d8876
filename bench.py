#!/usr/bin/env python
"""Benchmark of the two hot paths on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline (`metric` / `value`): fused linear-cross-entropy forward+backward tokens/s at
N=8192, D=4096, V=151936, bf16 (3 % of rows ignore_index), d_hidden with fp32 accumulation.
A "step" is one forward + one backward over that batch with the inputs already resident in
HBM.  The inputs are the seeded tensors of `configs.ce_dense(..., seed=0)`, drawn on the CPU:
the same tensors the full-size parity test feeds the kernels.  At N GPUs the lm_head is
vocab-sharded V/N per rank (strong scaling: the problem is fixed): forward partial triples are
all-gathered and the fp32 partial d_hidden is all-reduced across ranks, both inside the timed
region.  After the timed region rank 0 checks `lse`,
`nll` and `d_hidden` of 16 sampled rows of the very tensors it timed against the CPU oracle
(`parity`; the run aborts when they leave the test tolerances).  `e2e` is the same step
through the public operator (`linear_cross_entropy(...).backward()`) with the hidden states
and targets copied from pinned host memory every step (double-buffered: the copy for step i+1
is issued on a side stream while step i computes) and the loss read back; d_hidden stays on
the device, where a trainer consumes it.

The `attention` object carries the second half of the metric: causal GQA flash attention
forward+backward TFLOP/s at S=8192, 32 q / 8 kv heads, d=128 (KV-head-group sharded at N>1,
no collective), with its own `e2e`, `cpu_baseline`, a per-kernel `roofline` list (forward, dQ,
dK/dV event-timed separately) and, at N=1, the sequence-length sweep.  `c3` (4-bit head) and
`c5` (packed 16384-token row: attention + loss) are the other benchmark configurations, N=1.

`--impl reference` times the CPU restatement of the reference's own chunked implementation
(the oracle; MLX itself cannot be installed here) on the host cores, rank 0 only.

One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import json
import math
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


def ce_backward_chunks(n: int, v_local: int) -> int:
    """Backward chunks the library makes of `v_local` vocab rows (for the launch count): the rows are
    spread over the fewest chunks of at most 16384 rows whose (N, chunk) bf16 tile fits 512 MiB."""
    bound = min(16384, max(2048, (512 << 20) // (2 * n) // 256 * 256))
    return -(-v_local // bound)

PARITY_ROWS = 16
# tolerances of the full-size parity tests
TOL_LSE_REL, TOL_NLL_REL, TOL_DH_REL = 2e-5, 2e-3, 1.5e-2

# dram__bytes_read.sum + dram__bytes_write.sum of one ce_logits_kernel<FWD> launch at N=8192,
# D=4096, V=32768 (128 vocab tiles) from an ncu capture of `bench.py --small`; the traffic is
# proportional to the vocab-tile count, so a full launch is this figure times tiles / 128.
CE_FWD_TRAFFIC_BYTES_V32768 = 1.615e9
# the same two counters for the three attention kernels at S=4096 (forward, dQ, dK/dV); the K / V
# re-reads hit L2, so the traffic is the tensors themselves and grows linearly with S
ATT_TRAFFIC_BYTES_S4096 = {"flash_fwd2_kernel": 54.6e6, "flash_dq_kernel": 137.9e6, "flash_dkv_kernel": 94.3e6}


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


def loop_ms(fn, iters: int, warm: int, device) -> float:
    """Mean device time of `fn` over `iters` back-to-back calls (CUDA events, current stream)."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize(device)
    return e0.elapsed_time(e1) / iters


def cpu_baseline_ce(w_cpu, hidden_cpu, targets_cpu, cotangent_cpu, budget_s: float = 15.0):
    """The oracle (a port of the reference's chunked path) on the host cores, on the first R
    rows of the same workload with the full vocabulary; R sized for about `budget_s` seconds."""
    from oracle import linear_ce as oc
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    w32 = w_cpu.float()

    def run(rows):
        t0 = time.perf_counter()
        _, lse, _ = oc.streamed_lse_and_target(hidden_cpu[:rows], w32, targets_cpu[:rows])
        oc.chunked_backward(hidden_cpu[:rows], w32, targets_cpu[:rows], lse, cotangent_cpu[:rows])
        return time.perf_counter() - t0

    probe = run(32)
    rows = int(max(32, min(2048, 32 * budget_s / max(probe, 1e-3))))
    rows = max(32, rows // 32 * 32)
    t = run(rows)
    return {"value": rows / t, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"first {rows} of {N_TOK} rows, full V={VOCAB}, fp32 torch-CPU, fwd+bwd, {t:.1f} s"}


def cpu_baseline_attention(inp):
    """The attention oracle (materialised fp32 forward + hand-written backward) on the host cores for
    ONE kv head and its query heads at the full sequence length, one query head at a time (an (S, S)
    fp32 matrix is 256 MB at S=8192).  The rate does not depend on how many groups are run."""
    from oracle import attention as oa
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    group = ATT_HQ // ATT_HKV
    s = inp.q.shape[2]
    t0 = time.perf_counter()
    for h in range(group):
        q, k, v, d_o = inp.q[:, h:h + 1], inp.k[:, :1], inp.v[:, :1], inp.d_o[:, h:h + 1]
        o, lse = oa.flash_attention_reference(q, k, v, scale=inp.scale)
        oa.flash_attention_backward(q, k, v, o.to(torch.bfloat16), lse, d_o, scale=inp.scale)
    t = time.perf_counter() - t0
    flops = 7.0 * group * float(s) * s * ATT_D
    return {"value": flops / t / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"one kv head + its {group} query heads of {ATT_HKV} kv heads at S={s} (1/{ATT_HKV} of the "
                      f"workload; the rate extrapolates), fp32 torch-CPU oracle fwd+bwd, {t:.1f} s"}


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
    calls = [0]

    def one():
        qk_norm_rope(xs[calls[0] % 3], cos, sin, weight=w)
        calls[0] += 1

    with torch.no_grad():
        ms = loop_ms(one, n, 5, device)
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


class HostPipeline:
    """Double-buffered host -> device input feed, as a training loop's data loader runs it: step
    i+1's copies from pinned memory are issued on a side stream while step i's kernels run; every
    step still copies its own inputs inside the timed region."""

    def __init__(self, device, host_tensors):
        self.device, self.host = device, host_tensors
        self.stream = torch.cuda.Stream(device=device)
        self.pending = None

    def _prefetch(self):
        with torch.cuda.stream(self.stream):
            out = [t.to(self.device, non_blocking=True) for t in self.host]
            ev = torch.cuda.Event()
            ev.record(self.stream)
        return out, ev

    def next(self):
        if self.pending is None:
            self.pending = self._prefetch()
        out, ev = self.pending
        main = torch.cuda.current_stream(self.device)
        main.wait_event(ev)
        for t in out:
            t.record_stream(main)
        self.pending = self._prefetch()
        return out

    @property
    def bytes_per_step(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.host)


def ce_parity(inp_cpu, lse, nll, dh, rank_note: str):
    """lse / nll / d_hidden of PARITY_ROWS sampled rows of the timed tensors against the CPU oracle
    (full vocabulary).  Returns the `parity` object; raises SystemExit outside the test tolerances."""
    from mlx_train_perf_b200 import configs
    from oracle import linear_ce as oc
    g = torch.Generator().manual_seed(1)
    rows = torch.randperm(inp_cpu.hidden.shape[0], generator=g)[:PARITY_ROWS].sort().values
    ign = (inp_cpu.targets == configs.IGNORE_INDEX).nonzero()
    if ign.numel():
        rows[0] = int(ign[0])      # include an ignored row
    hs, ts, cs = inp_cpu.hidden[rows], inp_cpu.targets[rows], inp_cpu.cotangent[rows]
    r_nll, r_lse, _ = oc.streamed_lse_and_target(hs, inp_cpu.weight, ts, chunk_size=16384)
    r_dh, _ = oc.chunked_backward(hs, inp_cpu.weight, ts, r_lse, cs, chunk_size=16384)
    lse_s, nll_s, dh_s = lse.cpu()[rows], nll.cpu()[rows], dh.float().cpu()[rows]
    valid = ts != configs.IGNORE_INDEX
    res = {"rows": int(rows.numel()), "against": "oracle.linear_ce (fp32 CPU, full V) on the timed tensors" + rank_note,
           "lse_max_abs": float((lse_s - r_lse).abs().max()),
           "lse_max_rel": float(((lse_s - r_lse).abs() / r_lse.abs()).max()),
           "nll_max_rel": float(((nll_s - r_nll).abs()[valid] / r_nll[valid]).max()),
           "dh_rel": float((dh_s - r_dh).abs().max() / r_dh.abs().max()),
           "ignored_rows_zero": bool((nll_s[~valid] == 0).all() and (dh_s[~valid] == 0).all()),
           "tolerances": {"lse_max_rel": TOL_LSE_REL, "nll_max_rel": TOL_NLL_REL, "dh_rel": TOL_DH_REL}}
    ok = (res["lse_max_rel"] < TOL_LSE_REL and res["nll_max_rel"] < TOL_NLL_REL and res["dh_rel"] < TOL_DH_REL
          and res["ignored_rows_zero"] and math.isfinite(res["dh_rel"]))
    res["ok"] = ok
    if not ok:
        sys.stderr.write("parity check failed: " + json.dumps(res) + "\n")
        raise SystemExit(3)
    return res


def attention_block(args, world, rank, local, device, pk):
    """Second half of the metric: C4 flash attention fwd+bwd; sweep and per-kernel figures."""
    from mlx_train_perf_b200 import configs, parallel
    from mlx_train_perf_b200.attention import api as A
    from mlx_train_perf_b200.core import loss as L

    def shard(inp):
        if world == 1:
            return tuple(x.contiguous() for x in (inp.q, inp.k, inp.v, inp.d_o))
        q, k, v = parallel.shard_heads(inp.q, inp.k, inp.v, world, rank)
        d_o = inp.d_o[:, parallel.head_shard(ATT_HKV, ATT_HQ, world, rank)[1]]
        return tuple(x.contiguous() for x in (q, k, v, d_o))

    def make_sets(s):
        """Rotating input sets that together exceed L2, so no step finds its inputs cached."""
        sets, set_bytes = [], 0
        for seed in range(ATT_SETS):
            inp = configs.attention(s, hq=ATT_HQ, hkv=ATT_HKV, d=ATT_D, seed=seed, device=device)
            sets.append(shard(inp))
            set_bytes = sum(x.numel() * x.element_size() for x in sets[-1])
            if (seed + 1) * set_bytes > 160e6 and seed >= 1:
                break
        return sets, set_bytes, inp.scale

    def capture(fn, nsets):
        """One CUDA graph per rotating input set around `fn(i)`; returns a replay-next callable.  At small
        per-GPU shapes (a third of a millisecond per step at 8 GPUs) the Python and ctypes work of a step
        approaches the device time, so the timed loops replay graphs: the same kernels, launched back to
        back whatever the host is doing."""
        graphs = []
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            for i in range(nsets):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    keep = fn(i)
                graphs.append((g, keep))
        torch.cuda.current_stream(device).wait_stream(side)
        calls = [0]

        def replay():
            graphs[calls[0] % nsets][0].replay()
            calls[0] += 1
        replay.graphs = graphs
        return replay

    def step_fn(sets, scale, segments=None):
        def fn(i):
            q, k, v, d_o = sets[i % len(sets)]
            o, lse = A.flash_fwd_raw(q, k, v, scale=scale, segments=segments)
            return A.flash_bwd_raw(q, k, v, o, lse, d_o, scale=scale, segments=segments)
        return fn

    def fwd_fn(sets, scale, segments=None):
        def fn(i):
            q, k, v, _ = sets[i % len(sets)]
            return A.flash_fwd_raw(q, k, v, scale=scale, segments=segments)
        return fn

    sets, set_bytes, scale = make_sets(ATT_S)
    for i in range(3):
        step_fn(sets, scale)(i)          # first calls: module load, function attributes
    torch.cuda.synchronize(device)
    att_step = capture(step_fn(sets, scale), len(sets))
    att_fwd = capture(fwd_fn(sets, scale), len(sets))
    est = loop_ms(att_step, 5, 3, device)
    att_sampler = ClockSampler(local) if rank == 0 else None
    if att_sampler:
        att_sampler.launch()
    # long enough (>= 1.2 s) for nvidia-smi to sample the clocks at every GPU count
    att_steps = max(args.steps * 10, int(math.ceil(1200.0 / max(est, 1e-3))))
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([att_steps], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        att_steps = int(t.item())
    att_ms, att_clocks = timed_region(att_step, att_steps, max(args.warmup, 10), world, device, att_sampler)
    L.check_device_status()
    a_fwd_ms = loop_ms(att_fwd, max(50, att_steps // 4), 10, device)

    # forward, dQ (with the row statistics), dK/dV; + the GQA reduce when dK/dV CTAs are per q head (small
    # grids); + the combine pass when the forward is split over keys
    q0_, k0_, v0_ = sets[0][:3]
    fwd_split = A.flash_fwd_workspace_bytes(q0_, k0_, v0_, scale=scale) > 0
    row_vec = q0_.shape[0] * q0_.shape[1] * q0_.shape[2] * 4
    # the statistics tile is 8 row vectors' worth; fp32 partials are 256 of them (else no reduce pass)
    dkv_partials = A.flash_bwd_workspace_bytes(q0_, k0_, v0_, scale=scale) > 16 * row_vec
    att_launches = 3 + int(fwd_split) + int(dkv_partials)
    hq_local = ATT_HQ // world
    tfl = configs.attn_flops(1, ATT_HQ, ATT_S, ATT_D) / (att_ms / 1e3) / 1e12

    # ---- per-kernel device times: the backward with only its dQ kernel (which also forms the row
    # statistics) / only its dK, dV kernel (after the stand-alone statistics pre-pass, timed alone and subtracted)
    saved = []
    for q, k, v, d_o in sets:
        o, lse = A.flash_fwd_raw(q, k, v, scale=scale)
        saved.append((q, k, v, o, lse, d_o))

    def bwd_part(parts):
        def fn(i):
            q, k, v, o, lse, d_o = saved[i % len(saved)]
            return A.flash_bwd_raw(q, k, v, o, lse, d_o, scale=scale, parts=parts)
        return fn

    it = max(50, min(400, att_steps // 4))
    d_ms = loop_ms(capture(bwd_part("stats"), len(saved)), it, 10, device)
    dq_ms = loop_ms(capture(bwd_part("dq"), len(saved)), it, 10, device)
    dkv_ms = loop_ms(capture(bwd_part("dkv"), len(saved)), it, 10, device) - d_ms
    del saved
    s2d = float(ATT_S) * ATT_S * ATT_D * hq_local
    mhz = att_clocks.get("sm_mhz") if att_clocks else None
    scale_s = ATT_S / 4096.0

    def kroof(name, ms, flops, note):
        tf = flops / (ms / 1e3) / 1e12
        return {"kernel": name, "launch_ms": ms, "bound": "tensor", "achieved": tf, "peak": pk["burst"],
                "unit": "TFLOP/s", "frac": tf / pk["burst"], "frac_of_sustained": tf / pk["sustained"],
                "algorithmic_flops": flops, "peak_source": pk["source"] + " burst (cuBLAS bf16, best of 10)",
                "sm_mhz_median": mhz,
                "traffic": (ATT_TRAFFIC_BYTES_S4096.get(name.split(" ")[0], 0.0) * scale_s / world) or None,
                "note": note}

    fwd_name = "flash_fwd2_kernel" + (" (key range split) + flash_fwd_combine_kernel" if fwd_split else "")
    rooflines = [
        kroof(fwd_name, a_fwd_ms, 2.0 * s2d, "S = Q K^T and O = P V on the causal half"),
        kroof("flash_dq_kernel", dq_ms, 3.0 * s2d,
              "3 of the kernel's 3 GEMMs counted (S and dP recomputed here AND in dK/dV: the pair executes 7 "
              "GEMMs for the 5 the model counts); includes the row statistics D = rowsum(dO * O)"),
        kroof("flash_dkv_kernel" + (" + dkv_reduce_kernel" if dkv_partials else ""), dkv_ms, 4.0 * s2d,
              "4 GEMMs executed; the model's share of the backward is 5 - 3 = 2 of them"),
    ]
    bwd_ms = att_ms - a_fwd_ms
    bwd_tf = 5.0 * s2d / (bwd_ms / 1e3) / 1e12
    fwd_tfl = 2.0 * s2d / (a_fwd_ms / 1e3) / 1e12

    # ---- e2e through the public operator: q, k, v, dO from pinned host memory every step
    host = [x.cpu().pin_memory() for x in sets[0]]
    pipe = HostPipeline(device, host)

    def att_e2e_step():
        q, k, v, d_o = pipe.next()
        q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)
        o, lse = A.flash_attention_with_lse(q, k, v, scale=scale)
        torch.autograd.backward(o, d_o)
        return float(lse.sum().item())

    e2e_steps = max(10, args.steps)
    e2e_ms, _ = timed_region(att_e2e_step, e2e_steps, 3, world, device)
    L.check_device_status()
    e2e = {"value": configs.attn_flops(1, ATT_HQ, ATT_S, ATT_D) / (e2e_ms / 1e3) / 1e12, "unit": "TFLOP/s",
           "ms_per_step": e2e_ms, "h2d_bytes_per_step": pipe.bytes_per_step, "d2h_bytes_per_step": 4,
           "note": "flash_attention(...) + backward through autograd; q, k, v, dO copied from pinned host memory "
                   "each step (double-buffered), sum(L) read back; O, dQ, dK, dV stay on the device"}
    del pipe, host

    att = {"metric": "flash_attn_fwd_bwd_tflops", "value": tfl, "unit": "TFLOP/s", "ms_per_step": att_ms,
           "fwd_ms": a_fwd_ms, "bwd_ms": bwd_ms,
           "config": {"workload": f"C4 causal GQA B=1 Hq={ATT_HQ} Hkv={ATT_HKV} S={ATT_S} d={ATT_D} bf16",
                      "parallelism": f"kv-head-group x{world}",
                      "l2": "%d rotating input sets, %.0f MB together (L2 is 126 MB)"
                            % (len(sets), len(sets) * set_bytes / 1e6)},
           "flops_model": "7*B*Hq*S^2*d",
           "frac_of_burst": tfl / world / pk["burst"], "frac_of_sustained": tfl / world / pk["sustained"],
           "fwd_tflops_per_gpu": fwd_tfl, "bwd_tflops_per_gpu": bwd_tf,
           "bwd_frac_of_burst": bwd_tf / pk["burst"],
           "roofline": rooflines[0], "rooflines": rooflines,
           "timing": "CUDA-graph replay (one graph per rotating input set), CUDA events around the replays",
           "e2e": e2e, "cpu_baseline": None,
           "steps": att_steps, "clocks": att_clocks, "gpu_launches": att_launches * att_steps}
    if world > 1 or args.small:
        return att

    # ---- N=1 only: CPU baseline, sequence-length sweep, packed row, pre-step
    if not args.no_cpu_baseline:
        att["cpu_baseline"] = cpu_baseline_attention(configs.attention(ATT_S, seed=0))
    del sets
    torch.cuda.empty_cache()
    sweep = []
    for s in (2048, 4096, 16384):
        ssets, sbytes, sscale = make_sets(s)
        iters = 60 if s <= 4096 else 12
        st = capture(step_fn(ssets, sscale), len(ssets))
        fw = capture(fwd_fn(ssets, sscale), len(ssets))
        ms = loop_ms(st, iters, 5, device)
        f_ms = loop_ms(fw, iters, 5, device)
        sweep.append({"S": s, "fwd_bwd_ms": ms, "fwd_ms": f_ms,
                      "tflops": configs.attn_flops(1, ATT_HQ, s, ATT_D) / (ms / 1e3) / 1e12,
                      "frac_of_burst": configs.attn_flops(1, ATT_HQ, s, ATT_D) / (ms / 1e3) / 1e12 / pk["burst"],
                      "input_sets": len(ssets), "steps": iters})
        del ssets, st, fw
        torch.cuda.empty_cache()
    att["sweep"] = sweep
    att["prestep"] = prestep_bandwidth(device, pk, args.steps)
    return att


def c5_block(args, device, pk, weight):
    """The packed 16384-token row: segment-masked attention fwd+bwd and the fused loss at N=16384."""
    from mlx_train_perf_b200 import configs
    from mlx_train_perf_b200.attention import api as A
    from mlx_train_perf_b200.attention.segments import PackedMask
    from mlx_train_perf_b200.core import loss as L
    from mlx_train_perf_b200.core.loss import DenseHead
    total = 16384
    lengths = configs.packed_lengths(total, seed=1)
    seg_id, seg_start = configs.segments_from_lengths(lengths, device)
    pm = PackedMask(seg_id=seg_id, seg_start=seg_start)
    sets = []
    for seed in (1, 2):
        inp = configs.attention(total, hq=ATT_HQ, hkv=ATT_HKV, d=ATT_D, seed=seed, device=device)
        sets.append((inp.q, inp.k, inp.v, inp.d_o))
    calls = [0]

    def att_step():
        q, k, v, d_o = sets[calls[0] % 2]
        calls[0] += 1
        o, lse = A.flash_fwd_raw(q, k, v, scale=inp.scale, segments=pm)
        A.flash_bwd_raw(q, k, v, o, lse, d_o, scale=inp.scale, segments=pm)

    a_ms = loop_ms(att_step, 20, 5, device)
    a_flops = configs.attn_flops(1, ATT_HQ, total, ATT_D, seg_lengths=lengths)
    del sets
    torch.cuda.empty_cache()
    g = torch.Generator(device=device)
    g.manual_seed(1)
    hidden = torch.randn(total, D_MODEL, generator=g, device=device).to(torch.bfloat16)
    targets = torch.randint(0, weight.shape[0], (total,), generator=g, device=device, dtype=torch.int64)
    ends = torch.tensor(lengths, device=device).cumsum(0) - 1
    targets[ends] = configs.IGNORE_INDEX
    valid = targets != configs.IGNORE_INDEX
    ct = valid.float() / valid.sum()
    head = DenseHead(weight=weight)

    def ce_step():
        _, _, _, lse, _ = L.ce_forward_raw(hidden, head, targets)
        L.ce_backward_raw(hidden, head, targets, lse, ct)

    c_ms = loop_ms(ce_step, 4, 2, device)
    L.check_device_status()
    return {"workload": f"C5 packed row, {total} tokens in {len(lengths)} segments of 128-4096 (numpy rng 1)",
            "attention_fwd_bwd_ms": a_ms, "attention_tflops": a_flops / (a_ms / 1e3) / 1e12,
            "attention_flops_model": "sum over segments of 7*Hq*L_i^2*d",
            "ce_ms_per_step": c_ms, "ce_tokens_per_s": total / (c_ms / 1e3),
            "ce_tflops": configs.ce_flops(total, D_MODEL, weight.shape[0]) / (c_ms / 1e3) / 1e12,
            "tokens_per_s_attention_plus_loss": total / ((a_ms + c_ms) / 1e3), "steps": {"attention": 20, "ce": 4}}


def c3_block(args, device, hidden, targets, cotangent):
    """The 4-bit affine group-64 head at the headline shape."""
    from mlx_train_perf_b200 import configs
    from mlx_train_perf_b200.core import loss as L
    from mlx_train_perf_b200.core.loss import QuantizedHead
    g = torch.Generator(device=device)
    g.manual_seed(0)
    v, d = VOCAB, D_MODEL
    words = torch.randint(-2 ** 31, 2 ** 31, (v, d // 8), generator=g, device=device, dtype=torch.int64).to(torch.int32)
    scales = (torch.randn(v, d // 64, generator=g, device=device) * 0.01).abs().to(torch.bfloat16)
    biases = (-8.0 * scales.float()).to(torch.bfloat16)
    head = QuantizedHead(w_q=words, scales=scales, biases=biases)

    def make_step(impl):
        def step():
            _, _, _, lse, _ = L.ce_forward_raw(hidden, head, targets, impl=impl)
            L.ce_backward_raw(hidden, head, targets, lse, cotangent, impl=impl)
        return step

    ms = loop_ms(make_step("auto"), 5, 2, device)
    inline_ms = loop_ms(make_step("tc_inline"), 3, 1, device)
    L.check_device_status()
    a, _ = L._ce_args(hidden, head, targets, v_offset=0, ignore_index=configs.IGNORE_INDEX, impl="auto")
    from mlx_train_perf_b200 import _lib
    import ctypes as C
    lib = _lib.load()
    return {"workload": f"C3 int4 group-64 head, N={N_TOK} D={D_MODEL} V={VOCAB}, codes uniform (random words), "
                        "scales |N(0,0.01)| bf16, biases -8 scale",
            "ms_per_step": ms, "tokens_per_s": N_TOK / (ms / 1e3),
            "tflops": configs.ce_flops(N_TOK, D_MODEL, VOCAB) / (ms / 1e3) / 1e12,
            "dequantisation": "chunk by chunk into a bf16 scratch ahead of the dense kernels (the library's choice "
                              "above 512 rows); the same step with the head expanded inside the kernels, which "
                              "repeats the expansion for every 128-row block of hidden, is `inline_ms_per_step`",
            "inline_ms_per_step": inline_ms, "inline_tokens_per_s": N_TOK / (inline_ms / 1e3),
            "fwd_workspace_bytes": int(lib.b200tp_linear_ce_fwd_workspace_bytes(C.byref(a))),
            "bwd_workspace_bytes": int(lib.b200tp_linear_ce_bwd_workspace_bytes(C.byref(a), _lib.BF16)),
            "steps": 5}


def aux_block(device, pk, iters: int = 10, warm: int = 3):
    """`--aux`: the secondary kernels of the two paths, each event-timed alone on inputs larger than
    L2 (or rotating over enough copies): the trainable head's dW product, the chunk-wise 4-bit
    dequantisation, the attention kernels a small per-GPU grid selects (single-tile and key-split
    forward with its combine pass, per-q-head dK/dV with its reduce pass), the RMSNorm + RoPE
    pre-step both ways and the loss reduction.  One JSON line; no headline metric."""
    import ctypes as C
    from mlx_train_perf_b200 import _lib, configs
    from mlx_train_perf_b200.attention.api import flash_bwd_raw, flash_fwd_raw
    from mlx_train_perf_b200.attention.prestep import qk_norm_rope
    from mlx_train_perf_b200.core import loss as L
    from mlx_train_perf_b200.core.loss import DenseHead, reduced_linear_cross_entropy
    lib = _lib.load()
    out = []
    g = torch.Generator(device=device)
    g.manual_seed(0)

    # ---- trainable dense head: one 16384-row chunk; dW = the difference to the frozen backward
    n, d, v = N_TOK, D_MODEL, 16384
    h = torch.randn(n, d, generator=g, device=device).to(torch.bfloat16)
    w = (torch.randn(v, d, generator=g, device=device) * d ** -0.5).to(torch.bfloat16)
    t = torch.randint(0, v, (n,), generator=g, device=device)
    ct = torch.full((n,), 1.0 / n, device=device)
    head = DenseHead(weight=w)
    lse = L.ce_forward_raw(h, head, t)[3]
    dw = torch.empty_like(w)
    frozen = loop_ms(lambda: L.ce_backward_raw(h, head, t, lse, ct), iters, warm, device)
    train = loop_ms(lambda: L.ce_backward_raw(h, head, t, lse, ct, d_weight=dw), iters, warm, device)
    fl = 2.0 * n * v * d
    out.append({"kernel": "ce_dw_kernel", "case": f"N={n} D={d} V={v} bf16, one chunk",
                "ms": train - frozen, "tflops": fl / ((train - frozen) / 1e3) / 1e12,
                "frac_of_burst": fl / ((train - frozen) / 1e3) / 1e12 / pk["burst"],
                "backward_frozen_ms": frozen, "backward_trainable_ms": train})
    del dw

    # ---- chunk-wise 4-bit dequantisation, 16384 x 4096 (33.5 MB of codes + 2 MB of parameters -> 134 MB)
    words = torch.randint(-2 ** 31, 2 ** 31, (v, d // 8), generator=g, device=device, dtype=torch.int64).to(torch.int32)
    sc = (torch.randn(v, d // 64, generator=g, device=device) * 0.01).abs().to(torch.bfloat16)
    bi = (-8 * sc.float()).to(torch.bfloat16)
    outs = [torch.empty(v, d, dtype=torch.bfloat16, device=device) for _ in range(3)]   # rotate: 400 MB > L2
    stream = torch.cuda.current_stream(device).cuda_stream
    it = [0]

    def dq():
        it[0] += 1
        _lib.check(lib.b200tp_dequant_int4(words.data_ptr(), sc.data_ptr(), bi.data_ptr(), _lib.BF16, 0, v, d, 64,
                                           outs[it[0] % 3].data_ptr(), _lib.BF16, stream))
    ms = loop_ms(dq, iters, warm, device)
    nbytes = v * d / 2 + 2 * v * (d // 64) * 2 + v * d * 2
    out.append({"kernel": "dequant_int4_kernel", "case": f"{v} x {d}, bf16 parameters, bf16 out", "ms": ms,
                "gbs": nbytes / (ms / 1e3) / 1e9, "frac_of_hbm": nbytes / (ms / 1e3) / 1e9 / pk["hbm"],
                "algorithmic_bytes": nbytes})
    del outs, words, sc, bi, h, w

    # ---- attention on the grid one GPU of eight sees: one kv head, four q heads, S=8192
    sets = []
    for i in range(12):
        inp = configs.attention(ATT_S, seed=i)
        sl = slice(0, 4)
        sets.append(tuple(x.to(device) for x in (inp.q[:, sl], inp.k[:, :1], inp.v[:, :1], inp.d_o[:, sl])))
    scale = ATT_D ** -0.5
    k_it = [0]

    def att(fn):
        def run():
            k_it[0] += 1
            fn(*sets[k_it[0] % len(sets)])
        return run
    saved = [flash_fwd_raw(q, k, v_, scale=scale) for q, k, v_, _ in sets]
    fl_f = configs.attn_flops(1, 4, ATT_S, ATT_D) * 2 / 7
    for impl, label in (("auto", "flash_fwd2_kernel (two shares per query block) + flash_fwd_combine_kernel"),
                        ("tc1", "flash_fwd_kernel (single tile per CTA)"), ("tc2", "flash_fwd2_kernel, unsplit")):
        ms = loop_ms(att(lambda q, k, v_, _d: flash_fwd_raw(q, k, v_, scale=scale, impl=impl)), iters, warm, device)
        out.append({"kernel": label, "case": f"B=1 Hq=4 Hkv=1 S={ATT_S} d={ATT_D}", "impl": impl, "ms": ms,
                    "tflops": fl_f / (ms / 1e3) / 1e12, "frac_of_burst": fl_f / (ms / 1e3) / 1e12 / pk["burst"]})

    def bwd(parts):
        def run():
            k_it[0] += 1
            i = k_it[0] % len(sets)
            q, k, v_, d_o = sets[i]
            flash_bwd_raw(q, k, v_, saved[i][0], saved[i][1], d_o, scale=scale, parts=parts)
        return run
    for parts, label, gemms in (("dq", "flash_dq_kernel (+ row statistics)", 3),
                                ("dkv", "bwd_d_kernel + flash_dkv_kernel (per-q-head CTAs) + dkv_reduce_kernel", 4)):
        ms = loop_ms(bwd(parts), iters, warm, device)
        fl_b = configs.attn_flops(1, 4, ATT_S, ATT_D) * gemms / 7
        out.append({"kernel": label, "case": f"B=1 Hq=4 Hkv=1 S={ATT_S} d={ATT_D}", "ms": ms,
                    "tflops": fl_b / (ms / 1e3) / 1e12, "frac_of_burst": fl_b / (ms / 1e3) / 1e12 / pk["burst"]})
    del sets, saved

    # ---- RMSNorm + RoPE pre-step, forward and backward, x (4, 8192, 32, 128) bf16 (268 MB)
    b_, l_, h_, d_ = 4, 8192, 32, 128
    xs = [torch.randn(b_, l_, h_, d_, generator=g, device=device).to(torch.bfloat16).requires_grad_(True)
          for _ in range(2)]
    wn = torch.ones(d_, device=device, dtype=torch.bfloat16).requires_grad_(True)
    pos = torch.arange(l_, device=device, dtype=torch.float32)[:, None]
    inv = 10000.0 ** (-torch.arange(0, d_, 2, device=device, dtype=torch.float32) / d_)
    emb = torch.cat((pos * inv, pos * inv), -1)
    cos, sin = emb.cos().to(torch.bfloat16).contiguous(), emb.sin().to(torch.bfloat16).contiguous()
    ys = [qk_norm_rope(x, cos, sin, weight=wn) for x in xs]
    gy = torch.randn_like(ys[0])
    fwd = loop_ms(lambda: qk_norm_rope(xs[0].detach(), cos, sin, weight=wn.detach()), iters, warm, device)
    i_ = [0]

    def pre_bwd():
        i_[0] += 1
        torch.autograd.grad(ys[i_[0] % 2], (xs[i_[0] % 2], wn), gy, retain_graph=True)
    bw = loop_ms(pre_bwd, iters, warm, device)
    xb = b_ * l_ * h_ * d_ * 2
    out.append({"kernel": "norm_rope_fwd_kernel", "case": f"x ({b_},{l_},{h_},{d_}) bf16", "ms": fwd,
                "gbs": 2 * xb / (fwd / 1e3) / 1e9, "frac_of_hbm": 2 * xb / (fwd / 1e3) / 1e9 / pk["hbm"]})
    out.append({"kernel": "norm_rope_bwd_kernel (+ the weight-gradient reduction)", "case": f"x ({b_},{l_},{h_},{d_}) bf16",
                "ms": bw, "gbs": 3 * xb / (bw / 1e3) / 1e9, "frac_of_hbm": 3 * xb / (bw / 1e3) / 1e9 / pk["hbm"],
                "algorithmic_bytes": 3 * xb})
    del xs, ys, gy

    # ---- masked mean of the per-row loss and its cotangent (launch-bound: 8192 rows)
    nll = torch.rand(N_TOK, device=device)
    tg = torch.randint(0, 100, (N_TOK,), device=device)
    o3 = torch.empty(3, device=device)
    ms = loop_ms(lambda: _lib.check(lib.b200tp_linear_ce_reduce(nll.data_ptr(), tg.data_ptr(), N_TOK, -100,
                                                                o3.data_ptr(), stream)), iters, warm, device)
    out.append({"kernel": "loss_reduce_kernel", "case": f"N={N_TOK}", "ms": ms})
    L.check_device_status()
    return out


def main():
    claim_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-attention", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the C3 / C5 blocks (N=1 only anyway)")
    ap.add_argument("--aux", action="store_true",
                    help="time the secondary kernels alone (one GPU) and print their figures instead of the metric")
    ap.add_argument("--small", action="store_true",
                    help="profiling case: V=32768 and S=4096 (inputs still exceed L2), no e2e / CPU legs / extras")
    args = ap.parse_args()
    global VOCAB, ATT_S
    if args.small:
        VOCAB, ATT_S = 32768, 4096
        args.no_cpu_baseline = True
        args.no_extras = True
    args.aux_warmup = args.warmup          # --aux takes the counts as given (a profiler wants few launches)
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
        return

    from mlx_train_perf_b200 import configs, parallel
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
    if args.aux:
        if world > 1:
            raise SystemExit("--aux is a one-GPU measurement")
        emit({"aux": aux_block(device, pk, args.steps, args.aux_warmup), "n_gpus": 1, "peaks": pk})
        return

    # ------------------------------------------------------------------ linear-CE workload
    # the seeded CPU tensors of the parity tests (every rank draws the same stream and keeps its shard)
    inp_cpu = configs.ce_dense(N_TOK, D_MODEL, VOCAB, dtype=torch.bfloat16, ignore_frac=0.03, seed=0)
    hidden, targets, cotangent = (x.to(device) for x in (inp_cpu.hidden, inp_cpu.targets, inp_cpu.cotangent))
    lo, hi = parallel.shard_bounds(VOCAB, world, rank)
    weight = inp_cpu.weight[lo:hi].to(device)
    if rank != 0:
        inp_cpu.weight = None     # only rank 0 runs the oracle
    head = DenseHead(weight=weight)
    v_local = hi - lo

    fwd_ms = []
    kept = {}

    if world == 1:
        def step():
            f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            f0.record()
            _, _, _, lse, nll = L.ce_forward_raw(hidden, head, targets)
            f1.record()
            kept["out"] = (lse, nll, L.ce_backward_raw(hidden, head, targets, lse, cotangent))
            fwd_ms.append((f0, f1))
    else:
        sharded = parallel.VocabShardedLinearCE(head, lo)

        def step():
            f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            f0.record()
            nll, lse, _ = sharded.forward(hidden, targets)
            f1.record()
            kept["out"] = (lse, nll, sharded.backward(hidden, targets, lse, cotangent))
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
    chunks = ce_backward_chunks(N_TOK, v_local)
    launches_per_step = 2 + 2 * chunks    # logits fwd + combine; (g, dH) per backward chunk
    fwd_flops = 2.0 * N_TOK * v_local * D_MODEL
    fwd_tflops = fwd_flops / (fwd_avg_ms / 1e3) / 1e12
    step_tflops = configs.ce_flops(N_TOK, D_MODEL, VOCAB) / (ms_step / 1e3) / 1e12 / world

    # ------------------------------------------------------------------ parity of the timed path (rank 0)
    parity = None
    if rank == 0:
        lse_o, nll_o, dh_o = kept["out"]
        parity = ce_parity(inp_cpu, lse_o, nll_o, dh_o,
                           "" if world == 1 else f"; vocab-sharded over {world} NCCL ranks")
    kept.clear()

    # ------------------------------------------------------------------ e2e through the public API
    e2e = None
    if not args.small:
        if world == 1:
            pipe = HostPipeline(device, [inp_cpu.hidden.pin_memory(), inp_cpu.targets.pin_memory()])

            def e2e_step():
                h, t = pipe.next()
                h.requires_grad_(True)
                loss = linear_cross_entropy(h, head, t, reduction="mean", validate_targets=False)
                loss.backward()
                return float(loss.item())
        else:
            import torch.distributed as dist
            rows = N_TOK // world
            pipe = HostPipeline(device, [inp_cpu.hidden[rank * rows:(rank + 1) * rows].clone().pin_memory(),
                                         inp_cpu.targets.pin_memory()])
            gathered = {}
            lag = {"i": 0, "last": float("nan"), "host": [torch.empty(1, dtype=torch.float32).pin_memory() for _ in range(2)],
                   "ev": [torch.cuda.Event() for _ in range(2)]}

            def gather_next():
                # every rank needs all rows (the vocabulary, not the batch, is sharded): copy 1/R of them
                # over PCIe and rebuild the batch over NVLink; issued one step ahead, like the H2D copy
                part, t = pipe.next()
                h = torch.empty((N_TOK, D_MODEL), dtype=part.dtype, device=device)
                work = dist.all_gather_into_tensor(h, part, async_op=True)
                gathered["next"] = (h, t, work, part)

            def e2e_step():
                if "next" not in gathered:
                    gather_next()
                h, t, work, _part = gathered.pop("next")
                work.wait()
                gather_next()
                nll, lse, _ = sharded.forward(h, t)
                loss, _count, ct = L.masked_loss(nll, t, mean=True)
                sharded.backward(h, t, lse, ct)
                # the 4-byte loss goes to pinned memory asynchronously and is read one step later (the way
                # a trainer logs it), so the host keeps enqueueing: at 3 ms per step a blocking read per
                # step would expose the enqueue time of the next one
                slot = lag["i"] % 2
                lag["i"] += 1
                lag["host"][slot].copy_(loss.reshape(1), non_blocking=True)
                lag["ev"][slot].record()
                if lag["i"] >= 2:
                    lag["ev"][1 - slot].synchronize()
                    lag["last"] = float(lag["host"][1 - slot])
                return lag["last"]

        e2e_ms, _ = timed_region(e2e_step, args.steps, args.warmup, world, device)
        if world > 1 and "next" in gathered:
            gathered.pop("next")[2].wait()
        if world > 1:
            torch.cuda.synchronize(device)
            if not math.isfinite(float(lag["host"][(lag["i"] - 1) % 2])):
                raise SystemExit("e2e: the loss read back from the device is not finite")
        L.check_device_status()
        e2e = {"value": N_TOK / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": pipe.bytes_per_step, "d2h_bytes_per_step": 4,
               "note": ("linear_cross_entropy(reduction='mean').backward(); hidden + targets from pinned host "
                        "memory each step, the 4-byte loss read back; d_hidden stays on the device for the trainer")
               if world == 1 else
                       ("VocabShardedLinearCE forward + masked_loss + backward; each rank copies 1/N of the rows from "
                        "pinned host memory and the batch is rebuilt by an NVLink all-gather, both one step ahead; "
                        "every step's 4-byte loss is copied to pinned memory and read by the host one step later")}
        del pipe

    # ------------------------------------------------------------------ CPU baseline (rank 0, N=1)
    cpu = None
    if world == 1 and rank == 0 and not args.no_cpu_baseline:
        cpu = cpu_baseline_ce(inp_cpu.weight, inp_cpu.hidden.float(), inp_cpu.targets, inp_cpu.cotangent)

    # ------------------------------------------------------------------ other configurations (N=1)
    c3 = c5 = None
    if world == 1 and not args.no_extras:
        c3 = c3_block(args, device, hidden, targets, cotangent)
        torch.cuda.empty_cache()
        c5 = c5_block(args, device, pk, weight)
        torch.cuda.empty_cache()

    # ------------------------------------------------------------------ attention workload
    att = None
    if not args.no_attention:
        del weight, head
        inp_cpu = None
        torch.cuda.empty_cache()
        att = attention_block(args, world, rank, local, device, pk)

    if rank == 0:
        line = {
            "metric": "linear_ce_fwd_bwd_tokens_per_s", "value": tokens_per_s, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": f"C2 fused linear-CE fwd+bwd(d_hidden) N={N_TOK} D={D_MODEL} V={VOCAB} bf16, "
                                   "3% ignore_index, fp32 accumulation",
                       "parallelism": f"vocab-sharded x{world}" if world > 1 else "single GPU",
                       "inputs": "configs.ce_dense(seed=0), drawn on the CPU (the parity test's tensors)",
                       "l2": "inputs exceed L2 (lm_head shard %.2f GB vs 126 MB)" % (v_local * D_MODEL * 2 / 1e9)},
            "roofline": {"bound": "tensor", "achieved": fwd_tflops, "peak": pk["sustained"], "unit": "TFLOP/s",
                         "frac": fwd_tflops / pk["sustained"],
                         "traffic": CE_FWD_TRAFFIC_BYTES_V32768 * (-(-v_local // 256)) / 128,
                         "kernel": "ce_logits_kernel<FWD> (+ the row combine kernel, a few microseconds)",
                         "launch_ms": fwd_avg_ms, "frac_of_burst": fwd_tflops / pk["burst"],
                         "peak_source": pk["source"] + " sustained (kernel timed inside a long step)"},
            "step_tflops_per_gpu": step_tflops, "step_frac_of_sustained": step_tflops / pk["sustained"],
            "step_frac_of_burst": step_tflops / pk["burst"],
            "flops_model": "6*N*V*D",
            "parity": parity,
            "cpu_baseline": cpu,
            "e2e": e2e,
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
            "c3": c3,
            "c5": c5,
            "attention": att,
        }
        emit(line)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
