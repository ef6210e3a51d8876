"""Sequence packer: first-fit packing of variable-length sequences into fixed-width rows with
per-position segment ids (host code, pure Python + numpy; yields torch tensors).

Behaviour follows src/mlx_train_perf/data/packing.py of the reference exactly (the
differential tests in tests/test_packing.py compare against vectors produced by the
reference's own functions): `pack_indices` :15-48, `pack_stats` :64-99, `build_row`
:102-156, `packed_iterate_batches` :159-254, batching analytics :265-387.

Row algebra.  A pack row is `pack_len + 1` tokens wide (the last column is target-only).
Each placed sequence costs `min(len, pack_len) + 1` slots: its tokens plus one zero pad slot
it owns.  On the `pack_len`-wide inputs axis every position belongs to exactly one segment
(the unused tail is its own last segment), so no attention row is ever fully masked.
Positions are NOT reset per segment (RoPE runs 0..pack_len).
"""
from __future__ import annotations

import random
from collections.abc import Iterator, Sequence
from dataclasses import dataclass
from typing import Any

import numpy as np
import torch

from mlx_train_perf_b200.errors import PackingError

OPEN_POOL = 8        # open packs scanned by first-fit before the oldest is closed
STOCK_PAD_TO = 32    # the unpacked baseline pads to 1 + 32 * ceil(max / 32)


def _slot_cost(length: int, pack_len: int) -> int:
    return min(length, pack_len) + 1


def pack_indices(lengths: Sequence[int], pack_len: int, *, seed: int, epoch: int) -> list[list[int]]:
    """Group dataset indices into packs; deterministic per (seed, epoch).

    Order: `random.Random(f"{seed}:{epoch}").shuffle`.  Placement: first open pack (oldest
    first, at most OPEN_POOL open) with room; a pack closes when at most one slot is left
    (the smallest sequence needs two)."""
    if pack_len < 1:
        raise PackingError(f"pack_len must be >= 1; got {pack_len}")
    if not lengths:
        raise PackingError("cannot pack an empty dataset")
    if any(n < 1 for n in lengths):
        raise PackingError("zero-length sequence in dataset")
    order = list(range(len(lengths)))
    random.Random(f"{seed}:{epoch}").shuffle(order)

    packs: list[list[int]] = []
    free: list[int] = []        # remaining slots per pack
    live: list[int] = []        # ids of packs still accepting sequences, oldest first
    for idx in order:
        need = _slot_cost(lengths[idx], pack_len)
        home = next((p for p in live if free[p] >= need), None)
        if home is None:
            packs.append([idx])
            free.append(pack_len + 1 - need)
            live.append(len(packs) - 1)
            if len(live) > OPEN_POOL:
                del live[0]
            continue
        packs[home].append(idx)
        free[home] -= need
        if free[home] <= 1:
            live.remove(home)
    return packs


@dataclass(frozen=True)
class PackStats:
    """Utilisation over a `pack_len`-token budget per row (not `pack_len + 1`): the three
    fractions sum to 1 + 1/pack_len."""
    real_tokens: int
    capacity_tokens: int
    utilization: float
    separator_fraction: float
    tail_pad_fraction: float


def pack_stats(packs: list[list[int]], lengths: Sequence[int], pack_len: int) -> PackStats:
    if pack_len < 1:
        raise PackingError(f"pack_len must be >= 1; got {pack_len}")
    if not packs:
        raise PackingError("cannot compute stats over an empty pack list")
    real = sum(min(lengths[i], pack_len) for pack in packs for i in pack)
    seps = sum(len(pack) for pack in packs)
    tail = len(packs) * (pack_len + 1) - real - seps
    cap = len(packs) * pack_len
    return PackStats(real_tokens=real, capacity_tokens=cap, utilization=real / cap,
                     separator_fraction=seps / cap, tail_pad_fraction=tail / cap)


def build_row(entries: list[tuple[list[int], int]], pack_len: int):
    """One packed row from `(tokens, offset)` entries in pack order.

    Returns `(row, seg_id, seg_start, loss_mask)`: row has `pack_len + 1` tokens (one 0 pad
    after each sequence); the other three are `pack_len` wide.  A segment spans its tokens
    and its pad slot (clipped to the inputs axis); leftover capacity forms one trailing
    segment.  Supervised window of a segment starting at t0 with n tokens:
    `[t0 + max(offset, 1) - 1, t0 + n - 1]`."""
    row = np.zeros(pack_len + 1, dtype=np.int64)
    seg_id = np.zeros(pack_len, dtype=np.int64)
    seg_start = np.zeros(pack_len, dtype=np.int64)
    loss_mask = np.zeros(pack_len, dtype=bool)
    at = 0
    for sid, (tokens, offset) in enumerate(entries):
        n = len(tokens)
        row[at:at + n] = tokens
        last = min(at + n, pack_len - 1)            # pad slot, clipped off the target-only column
        seg_id[at:last + 1] = sid
        seg_start[at:last + 1] = at
        loss_mask[at + max(offset, 1) - 1:at + n] = True
        at += n + 1
    if at < pack_len:
        seg_id[at:] = len(entries)
        seg_start[at:] = at
    return row.tolist(), seg_id.tolist(), seg_start.tolist(), loss_mask.tolist()


def packed_iterate_batches(dataset: Any, batch_size: int, max_seq_length: int, loop: bool = False,
                           seed: int | None = None, comm_group: Any = None, *,
                           max_position_embeddings: int | None = None, device=None
                           ) -> Iterator[tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]]:
    """Batch iterator with the signature of mlx-lm's `iterate_batches`
    (data/packing.py:159-254): yields `(batch, seg_id, seg_start, loss_mask)` =
    int32 (B, L+1), int32 (B, L), int32 (B, L), bool (B, L), L = max_seq_length, identical
    shapes every step.  `dataset[j]` is `(tokens, offset)` or bare tokens.  Overlong sequences
    are truncated with one warning.  A trailing partial batch is dropped; `loop=True` reshuffles
    per epoch.

    Refuses (`PackingError`): a `comm_group` of size > 1 (pack on one worker and scatter);
    `max_seq_length > max_position_embeddings`; fewer packs than `batch_size`."""
    if comm_group is not None and comm_group.size() > 1:
        raise PackingError("packed_iterate_batches does not support distributed packing "
                           f"(comm_group.size()={comm_group.size()}); pack on a single worker")
    if max_position_embeddings is not None and max_seq_length > max_position_embeddings:
        raise PackingError(f"max_seq_length={max_seq_length} exceeds max_position_embeddings="
                           f"{max_position_embeddings}")
    items: list[tuple[list[int], int]] = []
    for j in range(len(dataset)):
        entry = dataset[j]
        if isinstance(entry, tuple) and len(entry) == 2:
            tokens, offset = entry
        else:
            tokens, offset = entry, 0
        items.append((list(tokens), int(offset)))
    longest = max((len(t) for t, _ in items), default=0)
    if longest > max_seq_length:
        print(f"[WARNING] Some sequences are longer than {max_seq_length} tokens. "
              f"The longest sentence {longest} will be truncated to {max_seq_length}. "
              "Consider pre-splitting your data to save memory.")
    items = [(t[:max_seq_length], o) for t, o in items]
    lengths = [len(t) for t, _ in items]

    epoch = 0
    while True:
        packs = pack_indices(lengths, max_seq_length, seed=seed or 0, epoch=epoch)
        full = len(packs) // batch_size
        if full == 0:
            raise PackingError(f"packed dataset produced {len(packs)} pack(s) at pack_len={max_seq_length}, "
                               f"fewer than batch_size={batch_size}; reduce batch_size or add more data")
        for b in range(full):
            built = [build_row([items[i] for i in pack], max_seq_length)
                     for pack in packs[b * batch_size:(b + 1) * batch_size]]
            rows, sids, ssts, masks = (np.array(x) for x in zip(*built))
            out = (torch.from_numpy(rows.astype(np.int32)), torch.from_numpy(sids.astype(np.int32)),
                   torch.from_numpy(ssts.astype(np.int32)), torch.from_numpy(masks.astype(bool)))
            yield tuple(t.to(device) for t in out) if device is not None else out
        epoch += 1
        if not loop:
            return


# ---------------------------------------------------------------------------------------
# dataset-level analytics (data/packing.py:265-387)
# ---------------------------------------------------------------------------------------
@dataclass(frozen=True)
class LengthHistogram:
    count: int
    mean: float
    median: float
    p90: float
    minimum: int
    maximum: int
    total_tokens: int


def length_histogram(lengths: Sequence[int]) -> LengthHistogram:
    if not lengths:
        raise PackingError("cannot summarize an empty length list")
    a = np.asarray(lengths, dtype=np.int64)
    return LengthHistogram(count=len(lengths), mean=float(a.mean()), median=float(np.median(a)),
                           p90=float(np.percentile(a, 90)), minimum=int(a.min()), maximum=int(a.max()),
                           total_tokens=int(a.sum()))


@dataclass(frozen=True)
class StockBatchingStats:
    num_batches: int
    real_tokens_total: int
    padded_tokens_total: int
    padding_waste_fraction: float
    mean_real_tokens_per_step: float
    mean_samples_per_step: float


def stock_batching_stats(lengths: Sequence[int], *, batch_size: int, max_seq_length: int) -> StockBatchingStats:
    """Padding waste of unpacked batching: sort by length, full batches only, each padded to
    min(1 + 32 * ceil(max_in_batch / 32), max_seq_length)."""
    if batch_size < 1:
        raise PackingError(f"batch_size must be >= 1; got {batch_size}")
    if max_seq_length < 1:
        raise PackingError(f"max_seq_length must be >= 1; got {max_seq_length}")
    ordered = sorted(lengths)
    real = padded = batches = 0
    for s in range(0, len(ordered) - batch_size + 1, batch_size):
        group = ordered[s:s + batch_size]
        width = min(1 + STOCK_PAD_TO * -(-group[-1] // STOCK_PAD_TO), max_seq_length)
        real += sum(min(n, max_seq_length) for n in group)
        padded += batch_size * width
        batches += 1
    return StockBatchingStats(num_batches=batches, real_tokens_total=real, padded_tokens_total=padded,
                              padding_waste_fraction=(padded - real) / padded if padded else 0.0,
                              mean_real_tokens_per_step=real / batches if batches else 0.0,
                              mean_samples_per_step=float(batch_size))


@dataclass(frozen=True)
class PackedBatchingStats:
    num_batches: int
    real_tokens_total: int
    mean_real_tokens_per_step: float
    mean_samples_per_step: float
    utilization: float
    separator_fraction: float
    tail_pad_fraction: float


def packed_batching_stats(lengths: Sequence[int], pack_len: int, *, batch_size: int, seed: int,
                          epoch: int = 0) -> PackedBatchingStats:
    """Per-step counts over the packs whole batches consume, plus whole-dataset utilisation."""
    if batch_size < 1:
        raise PackingError(f"batch_size must be >= 1; got {batch_size}")
    packs = pack_indices(lengths, pack_len, seed=seed, epoch=epoch)
    nb = len(packs) // batch_size
    used = packs[:nb * batch_size]
    real = sum(min(lengths[i], pack_len) for pack in used for i in pack)
    samples = sum(len(pack) for pack in used)
    st = pack_stats(packs, lengths, pack_len)
    return PackedBatchingStats(num_batches=nb, real_tokens_total=real,
                               mean_real_tokens_per_step=real / nb if nb else 0.0,
                               mean_samples_per_step=samples / nb if nb else 0.0,
                               utilization=st.utilization, separator_fraction=st.separator_fraction,
                               tail_pad_fraction=st.tail_pad_fraction)
