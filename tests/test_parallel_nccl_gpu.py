"""`VocabShardedLinearCE` over real NCCL ranks (two GPUs; skipped on a one-GPU machine): the sharded forward
and every form of the d_hidden reduction (plain all-reduce, reduce-scatter + 16-bit all-gather, staged)
against the CPU oracle and against each other.  Child processes, one per GPU, NVLS off (a plain ring is
enough for a parity test)."""
import os
import sys
from pathlib import Path

import pytest
import torch
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import datetime
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=120))
    from mlx_train_perf_b200 import configs, parallel
    from mlx_train_perf_b200.core import loss as L
    from oracle import linear_ce as oc
    n, d, v = 512, 256, 5003
    inp = configs.ce_dense(n, d, v, dtype=torch.bfloat16, ignore_frac=0.1, seed=31)
    h, t, ct = inp.hidden.to(dev), inp.targets.to(dev), inp.cotangent.to(dev)
    head, lo = parallel.shard_dense_head(inp.weight.to(dev), world, rank)
    outs = {}
    for name, kw in (("all_reduce", {}), ("scatter_gather", {"reduce_mode": "scatter_gather"}),
                     ("staged", {"reduce_stages": 2})):
        op = parallel.VocabShardedLinearCE(head, lo, **kw)
        nll, lse, tgt = op.forward(h, t)
        dh = op.backward(h, t, lse, ct)
        torch.cuda.synchronize()
        outs[name] = (nll.cpu(), lse.cpu(), dh.float().cpu())
    L.check_device_status()
    if rank == 0:
        ref_nll, ref_lse, _ = oc.naive_linear_ce(inp.hidden, inp.weight, inp.targets)
        ref_dh, _ = oc.chunked_backward(inp.hidden, inp.weight, inp.targets, ref_lse, inp.cotangent)
        for name, (nll, lse, dh) in outs.items():
            assert (lse - ref_lse).abs().max().item() < 1e-5, name
            assert (nll - ref_nll).abs().max().item() < 1e-5, name
            rel = (dh - ref_dh).abs().max().item() / ref_dh.abs().max().item()
            assert rel < 1.5e-2, (name, rel)
        # the staged form reduces the same fp32 partials in the same order: bit for bit the plain result
        assert torch.equal(outs["staged"][2], outs["all_reduce"][2])
        rel = (outs["scatter_gather"][2] - outs["all_reduce"][2]).abs().max().item() / ref_dh.abs().max().item()
        assert rel < 4e-3, rel      # another summation order before the single rounding: one bf16 ulp at most
    Path(out_dir, f"ok{rank}").write_text("ok")
    dist.destroy_process_group()


def test_vocab_sharded_loss_over_nccl(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    port = 29600 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()
