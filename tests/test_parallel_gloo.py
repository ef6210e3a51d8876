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
    for v, w in ((151936, 8), (151936, 4), (1001, 3), (8, 8)):
        spans = [parallel.shard_bounds(v, w, r) for r in range(w)]
        assert spans[0][0] == 0 and spans[-1][1] == v
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [b - a for a, b in spans]
        assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        parallel.head_shard(8, 32, 3, 0)
    # fewer vocab rows than ranks: refused identically on every rank (no rank may sit out of the all-gather)
    from mlx_train_perf_b200.errors import LossInputError
    for r in range(8):
        with pytest.raises(LossInputError):
            parallel.shard_bounds(7, 8, r)
    with pytest.raises(LossInputError):
        parallel.shard_dense_head(torch.zeros(3, 16), 4, 0)


def test_sharded_operator_validates_before_any_native_call():
    """`VocabShardedLinearCE` hands raw addresses to the kernels, so it runs the single-GPU operator's
    checks first: shape, dtype and device of every operand (CPU tensors never reach the library)."""
    from mlx_train_perf_b200 import parallel
    from mlx_train_perf_b200.core.loss import DenseHead
    from mlx_train_perf_b200.errors import LossInputError
    op = parallel.VocabShardedLinearCE(DenseHead(weight=torch.zeros(32, 16)), 0)
    h, t = torch.zeros(4, 16), torch.zeros(4, dtype=torch.int64)
    with pytest.raises(LossInputError, match="CUDA"):
        op.forward(h, t)                                  # a host tensor is refused, not dereferenced
    with pytest.raises(LossInputError, match="targets shape"):
        op.forward(h, torch.zeros(5, dtype=torch.int64))
    with pytest.raises(LossInputError, match="integer"):
        op.backward(h, t.float(), torch.zeros(4), torch.zeros(4))
    with pytest.raises(LossInputError, match="dtype"):
        op.forward(h.to(torch.bfloat16), t)
    with pytest.raises(ValueError, match="reduce_mode"):
        parallel.VocabShardedLinearCE(DenseHead(weight=torch.zeros(32, 16)), 0, reduce_mode="ring")
