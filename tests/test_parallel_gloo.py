"""Host-side logic of the multi-GPU forms on CPU ranks (gloo, world size 2): shard bounds, the
(R, 3, N) gather layout, the combine arithmetic and the partial-d_hidden reduction.  The
per-rank partials come from the oracle here; on GPUs they come from the kernels."""
import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from mlx_train_perf_b200 import configs, parallel
    from oracle import linear_ce as oc
    inp = configs.ce_dense(50, 32, 1001, dtype=torch.float32, ignore_frac=0.1, seed=7)
    lo, hi = parallel.shard_bounds(1001, world, rank)
    m, s, t = oc.shard_partials(inp.hidden, inp.weight[lo:hi], inp.targets, lo)
    parts = parallel.gather_partials(torch.stack((m, s, t)))
    assert tuple(parts.shape) == (world, 3, 50)
    nll, lse, tgt = parallel.combine_partials_reference(parts, inp.targets)
    ref = oc.naive_linear_ce(inp.hidden, inp.weight, inp.targets)
    for a, b in zip((nll, lse, tgt), ref):
        assert (a - b).abs().max().item() < 2e-6
    dh_part, _ = oc.chunked_backward(inp.hidden, inp.weight[lo:hi], inp.targets - lo, lse, inp.cotangent)
    # targets outside the shard never match a column; ignored rows must stay masked
    ign = inp.targets == configs.IGNORE_INDEX
    dh_part[ign] = 0
    dist.all_reduce(dh_part)
    dh_ref, _ = oc.chunked_backward(inp.hidden, inp.weight, inp.targets, ref[1], inp.cotangent)
    assert (dh_part - dh_ref).abs().max().item() < 1e-6
    # attention head sharding covers every head exactly once
    ks, qs = parallel.head_shard(8, 32, world, rank)
    cover = torch.zeros(32)
    cover[qs] = 1
    dist.all_reduce(cover)
    assert bool((cover == 1).all()) and ks == slice(rank * 4, rank * 4 + 4)
    Path(out_dir, f"ok{rank}").write_text("ok")
    dist.destroy_process_group()


def test_vocab_shard_combine_and_head_shards_world2(tmp_path):
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()


def test_shard_bounds_partition():
    from mlx_train_perf_b200 import parallel
    for v, w in ((151936, 8), (151936, 4), (1001, 3), (7, 8)):
        spans = [parallel.shard_bounds(v, w, r) for r in range(w)]
        assert spans[0][0] == 0 and spans[-1][1] == v
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [b - a for a, b in spans]
        assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        parallel.head_shard(8, 32, 3, 0)
