"""Multi-GPU forms of the two paths: one process per GPU, `torch.distributed` for plumbing.

The reference is single-device (its packer refuses a distributed group,
src/mlx_train_perf/data/packing.py:193-197); this module is new work.

* `VocabShardedLinearCE` -- rank r holds rows [r V/R, (r+1) V/R) of the lm_head and the full
  hidden states.  Forward: each rank's kernels emit per-row (max, sum-exp, target-logit)
  partials; ONE all-gather of an (N, 3) fp32 buffer (96 KiB per rank at N = 8192) and a tiny
  combine kernel give lse / nll on every rank.  Backward: each rank's kernels produce an fp32
  partial d_hidden over its shard, the partials are all-reduced (the one exchange the path
  really has: the hidden states are replicated, the vocabulary is not) and cast once.  The
  reduction is overlapped with the computation: the last vocab chunk's d_hidden GEMM is issued in
  a few slabs of finished rows (`b200tp_linear_ce_bwd_stage`), and each slab is all-reduced and
  cast on a side stream while the next one computes.
* `shard_heads` -- attention sharded by KV-head group: rank r owns KV heads
  [r Hkv/R, (r+1) Hkv/R) and their query heads; heads are independent and the GQA group sum
  stays on the rank, so the op needs no collective.

Works with the `nccl` backend on GPUs and (host logic only: shard bounds, gather layout,
combine arithmetic through `combine_partials_reference`) with `gloo` on CPU.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from mlx_train_perf_b200.core import loss as L
from mlx_train_perf_b200.core.loss import DenseHead, HeadRef, QuantizedHead
from mlx_train_perf_b200.errors import LossInputError

IGNORE_INDEX = L.IGNORE_INDEX


def shard_bounds(v: int, world: int, rank: int) -> tuple[int, int]:
    """Vocab rows [lo, hi) of rank `rank`: even split, the first v % world ranks get one more.
    Every rank must own at least one row (a rank with none would refuse its launch while the others
    wait for it in the all-gather), so V < world is refused here, identically on every rank."""
    if world < 1 or not 0 <= rank < world:
        raise LossInputError(f"rank {rank} is not in [0, {world})")
    if v < world:
        raise LossInputError(f"cannot shard V={v} vocab rows over {world} ranks: every rank needs at least one row")
    base, extra = divmod(v, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def head_shard(hkv: int, hq: int, world: int, rank: int) -> tuple[slice, slice]:
    """(kv-head slice, q-head slice) of rank `rank` under KV-head-group sharding."""
    if hkv % world != 0:
        raise ValueError(f"Hkv={hkv} must be divisible by the world size {world}")
    per = hkv // world
    group = hq // hkv
    return slice(rank * per, (rank + 1) * per), slice(rank * per * group, (rank + 1) * per * group)


def shard_heads(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, world: int, rank: int):
    """Views of this rank's heads of (B, H, S, d) tensors."""
    ks, qs = head_shard(k.shape[1], q.shape[1], world, rank)
    return q[:, qs], k[:, ks], v[:, ks]


def combine_partials_reference(parts: torch.Tensor, targets: torch.Tensor, ignore_index: int = IGNORE_INDEX):
    """Torch restatement of the combine kernel for parts (R, 3, N): used by the CPU (gloo)
    tests of the gather layout; the GPU path calls the library's combine kernel."""
    m = parts[:, 0].max(dim=0).values
    s = (parts[:, 1] * torch.exp(parts[:, 0] - m)).sum(dim=0)
    lse = m + torch.log(s)
    tgt = parts[:, 2].sum(dim=0)
    valid = targets != ignore_index
    tgt = torch.where(valid, tgt, torch.zeros_like(tgt))
    return torch.where(valid, lse - tgt, torch.zeros_like(lse)), lse, tgt


def gather_partials(local: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather a (3, N) fp32 partial buffer into (R, 3, N)."""
    world = dist.get_world_size(group)
    out = torch.empty(world * local.numel(), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out, local.contiguous().reshape(-1), group=group)
    return out.reshape((world,) + tuple(local.shape))


class VocabShardedLinearCE:
    """Forward/backward of the fused loss with the lm_head sharded over the vocabulary.

    `head` is THIS rank's shard (DenseHead or QuantizedHead over rows [lo, hi)); `v_offset` =
    lo.  `forward` returns (nll, lse, tgt) replicated on every rank; `backward` returns the
    full d_hidden (hidden dtype) replicated on every rank.

    `reduce_stages` > 1 issues the backward in that many stages and all-reduces each finished slab of
    rows on a side stream while the next slab computes.  It is off by default: the loss kernels are
    persistent and fill every SM's shared memory, so NCCL's reduction kernels only get SMs between
    launches and then hold their peers waiting -- measured on 4 GPUs at 18992 vocab rows per rank:
    3.32 ms per step unstaged, 3.54 ms with three stages, 3.84 ms with seven."""

    def __init__(self, head: HeadRef, v_offset: int, *, group=None, ignore_index: int = IGNORE_INDEX,
                 impl: str = "auto", reduce_stages: int = 1, reduce_mode: str = "all_reduce"):
        if reduce_mode not in ("scatter_gather", "all_reduce"):
            raise ValueError(f"unknown reduce_mode {reduce_mode!r}; expected 'scatter_gather' or 'all_reduce'")
        self.head, self.v_offset, self.group = head, int(v_offset), group
        self.ignore_index, self.impl = ignore_index, impl
        self.reduce_stages = max(1, int(reduce_stages))
        self.reduce_mode = reduce_mode
        self._side = None

    def _normalise(self, hidden: torch.Tensor, targets: torch.Tensor):
        """The checks and layout fixes the single-GPU operator applies before it hands raw addresses
        to the kernels: (N, D) contiguous hidden states of the head's dtype on a GPU, int64 targets."""
        if hidden.ndim != 2:
            raise LossInputError(f"hidden must be (N, D); got shape {tuple(hidden.shape)}")
        L._validate_inputs(hidden, self.head, targets, validate_targets=False, ignore_index=self.ignore_index)
        L._require_cuda(hidden, "hidden")
        if not hidden.is_contiguous():
            hidden = hidden.contiguous()
        return hidden, targets.reshape(-1).to(device=hidden.device, dtype=torch.int64).contiguous()

    def forward(self, hidden: torch.Tensor, targets: torch.Tensor):
        from mlx_train_perf_b200 import _lib
        hidden, targets = self._normalise(hidden, targets)
        n = hidden.shape[0]
        buf = L.ce_forward_buffer(hidden, self.head, targets, v_offset=self.v_offset,
                                  ignore_index=self.ignore_index, impl=self.impl, want_lse=False)
        local = buf[:3]   # (max, sum-exp, target logit): this rank's message
        parts = gather_partials(local, self.group)
        out = torch.empty((3, n), dtype=torch.float32, device=hidden.device)
        lib = _lib.load()
        with torch.cuda.device(hidden.device):
            rc = lib.b200tp_linear_ce_combine(parts.data_ptr(), parts.shape[0], n, targets.data_ptr(),
                                              self.ignore_index, out[0].data_ptr(), out[1].data_ptr(),
                                              out[2].data_ptr(),
                                              torch.cuda.current_stream(hidden.device).cuda_stream)
        _lib.check(rc)
        return out[1], out[0], out[2]   # nll, lse, tgt

    def backward(self, hidden: torch.Tensor, targets: torch.Tensor, lse: torch.Tensor, cotangent: torch.Tensor,
                 d_weight: torch.Tensor | None = None):
        """d_hidden (summed over the shards).  `d_weight`, shaped like this rank's weight shard,
        receives the shard's rows of the head gradient: they are disjoint across ranks, so
        no collective touches them."""
        hidden, targets = self._normalise(hidden, targets)
        if d_weight is not None or self.reduce_stages == 1:
            partial = L.ce_backward_raw(hidden, self.head, targets, lse, cotangent, v_offset=self.v_offset,
                                        ignore_index=self.ignore_index, impl=self.impl, out_dtype=torch.float32,
                                        d_weight=d_weight)
            return self._reduce(partial, hidden.dtype)
        return self._backward_overlapped(hidden, targets, lse, cotangent)

    def _reduce(self, partial: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        """Sum of the ranks' fp32 partial d_hidden, rounded once to `out_dtype`, on every rank.  With
        16-bit hidden states and rows that divide over the ranks: reduce-scatter in fp32, cast the owned
        rows, all-gather them in 16 bits -- the same sum and the same single rounding as an fp32 all-reduce
        followed by a cast, with three quarters of its traffic and no separate pass over the full matrix."""
        world = dist.get_world_size(self.group)
        n, d = partial.shape
        if self.reduce_mode == "all_reduce" or out_dtype == torch.float32 or n % world != 0:
            dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=self.group)
            return partial.to(out_dtype)
        own = torch.empty((n // world, d), dtype=torch.float32, device=partial.device)
        dist.reduce_scatter_tensor(own, partial, op=dist.ReduceOp.SUM, group=self.group)
        out = torch.empty((n, d), dtype=out_dtype, device=partial.device)
        dist.all_gather_into_tensor(out, own.to(out_dtype), group=self.group)
        return out

    def _backward_overlapped(self, hidden, targets, lse, cotangent):
        """The fp32 partial d_hidden is produced in `reduce_stages` slabs of rows; each finished slab
        is all-reduced and cast to the hidden dtype on a side stream while the kernels of the next slab
        run on the caller's stream.  Only the last slab's reduction is exposed."""
        from mlx_train_perf_b200 import _lib
        lib = _lib.load()
        dev = hidden.device
        n, d = hidden.shape
        a, keep = L._ce_args(hidden, self.head, targets, v_offset=self.v_offset, ignore_index=self.ignore_index,
                             impl=self.impl)
        partial = torch.empty((n, d), dtype=torch.float32, device=dev)
        out = torch.empty((n, d), dtype=hidden.dtype, device=dev)
        lse32 = lse.to(torch.float32).contiguous()
        ct = cotangent.to(torch.float32).contiguous()
        nbytes = lib.b200tp_linear_ce_bwd_workspace_bytes(C.byref(a), _lib.F32)
        ws = L._workspace(nbytes, dev)
        main = torch.cuda.current_stream(dev)
        if self._side is None:
            self._side = torch.cuda.Stream(device=dev)
        side = self._side
        rows_done = C.c_int64(0)
        prev = 0
        for stage in range(self.reduce_stages):
            with torch.cuda.device(dev):
                rc = lib.b200tp_linear_ce_bwd_stage(C.byref(a), lse32.data_ptr(), ct.data_ptr(), partial.data_ptr(),
                                                    _lib.F32, 0, self.reduce_stages, stage, C.byref(rows_done),
                                                    L._ptr(ws), nbytes, main.cuda_stream,
                                                    L.device_status(dev).data_ptr())
            _lib.check(rc)
            r1 = int(rows_done.value)
            if r1 > prev:
                ev = torch.cuda.Event()
                ev.record(main)
                side.wait_event(ev)
                with torch.cuda.stream(side):
                    slab = partial[prev:r1]
                    dist.all_reduce(slab, op=dist.ReduceOp.SUM, group=self.group)
                    out[prev:r1].copy_(slab)
                prev = r1
        main.wait_stream(side)
        for t in (partial, out, lse32, ct, ws):
            if t is not None:
                t.record_stream(side)
        del keep
        return out


def shard_dense_head(weight: torch.Tensor, world: int, rank: int) -> tuple[DenseHead, int]:
    """This rank's rows of a dense head and their vocab offset (refuses V < world on every rank)."""
    lo, hi = shard_bounds(weight.shape[0], world, rank)
    return DenseHead(weight=weight[lo:hi].contiguous()), lo


def shard_quantized_head(head: QuantizedHead, world: int, rank: int) -> tuple[QuantizedHead, int]:
    lo, hi = shard_bounds(head.w_q.shape[0], world, rank)
    return QuantizedHead(w_q=head.w_q[lo:hi].contiguous(), scales=head.scales[lo:hi].contiguous(),
                         biases=head.biases[lo:hi].contiguous(), group_size=head.group_size, bits=head.bits), lo
