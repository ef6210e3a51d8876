"""Packer: differential tests against vectors produced by the reference's own
`pack_indices` / `build_row` / `pack_stats` / batching analytics (tests/golden/packing.json,
written by tests/golden/make_host_golden.py), the reference's worked example
(tests/test_packing.py:106-119) and its properties (:10-21, :76-103, :127-159, :177-201)."""
import json
from pathlib import Path

import pytest
import torch
from hypothesis import given, settings
from hypothesis import strategies as st

from mlx_train_perf_b200.data import packing as P
from mlx_train_perf_b200.errors import PackingError

GOLD = json.loads((Path(__file__).parent / "golden" / "packing.json").read_text())


def test_pack_indices_and_stats_match_reference_vectors():
    n = 0
    for c in GOLD["cases"]:
        if c["kind"] != "pack":
            continue
        packs = P.pack_indices(c["lengths"], c["pack_len"], seed=c["seed"], epoch=c["epoch"])
        assert packs == c["packs"]
        s = P.pack_stats(packs, c["lengths"], c["pack_len"])
        for k, v in c["stats"].items():
            assert getattr(s, k) == pytest.approx(v, rel=1e-12)
        n += 1
    assert n >= 12


def test_batching_analytics_match_reference_vectors():
    for c in GOLD["cases"]:
        if c["kind"] != "batching":
            continue
        a = P.stock_batching_stats(c["lengths"], batch_size=c["batch_size"], max_seq_length=c["pack_len"])
        b = P.packed_batching_stats(c["lengths"], c["pack_len"], batch_size=c["batch_size"], seed=1)
        h = P.length_histogram(c["lengths"])
        for got, want in ((a, c["stock"]), (b, c["packed"]), (h, c["hist"])):
            for k, v in want.items():
                assert getattr(got, k) == pytest.approx(v, rel=1e-12), k


def test_build_row_matches_reference_vectors():
    for r in GOLD["rows"]:
        entries = [(list(t), o) for t, o in r["entries"]]
        row, sid, sst, mask = P.build_row(entries, r["pack_len"])
        assert row == r["row"] and sid == r["seg_id"] and sst == r["seg_start"] and mask == r["loss_mask"]


def test_build_row_worked_example():
    # two sequences (3 tokens offset 0, 2 tokens offset 1) in an 8-wide pack
    row, sid, sst, mask = P.build_row([([11, 12, 13], 0), ([21, 22], 1)], 8)
    assert row == [11, 12, 13, 0, 21, 22, 0, 0, 0]
    assert sid == [0, 0, 0, 0, 1, 1, 1, 2]
    assert sst == [0, 0, 0, 0, 4, 4, 4, 7]
    assert mask == [True, True, True, False, True, True, False, False]


@settings(max_examples=60, deadline=None)
@given(st.lists(st.integers(1, 300), min_size=1, max_size=80), st.integers(1, 256), st.integers(0, 5),
       st.integers(0, 3))
def test_pack_properties(lengths, pack_len, seed, epoch):
    packs = P.pack_indices(lengths, pack_len, seed=seed, epoch=epoch)
    flat = sorted(i for p in packs for i in p)
    assert flat == list(range(len(lengths)))                      # every index exactly once
    for p in packs:
        assert sum(min(lengths[i], pack_len) + 1 for i in p) <= pack_len + 1
    assert packs == P.pack_indices(lengths, pack_len, seed=seed, epoch=epoch)   # deterministic
    s = P.pack_stats(packs, lengths, pack_len)
    assert s.utilization + s.separator_fraction + s.tail_pad_fraction == pytest.approx(1 + 1 / pack_len)


@settings(max_examples=40, deadline=None)
@given(st.lists(st.tuples(st.integers(1, 20), st.integers(0, 25)), min_size=1, max_size=6))
def test_build_row_invariants(spec):
    pack_len = sum(n + 1 for n, _ in spec) + 3
    entries = [(list(range(1, n + 1)), off) for n, off in spec]
    row, sid, sst, mask = P.build_row(entries, pack_len)
    assert len(row) == pack_len + 1 and len(sid) == len(sst) == len(mask) == pack_len
    assert sid[0] == 0 and all(b - a in (0, 1) for a, b in zip(sid, sid[1:]))    # gapless, ascending
    assert all(a <= b for a, b in zip(sst, sst[1:]))
    assert all(sst[i] <= i and sid[sst[i]] == sid[i] for i in range(pack_len))
    assert not any(mask[i] for i in range(pack_len) if sid[i] == len(entries))    # tail is never supervised


class _Group:
    def __init__(self, n):
        self.n = n

    def size(self):
        return self.n


def test_iterate_batches_shapes_refusals_and_determinism(capsys):
    data = [(list(range(1, n + 1)), 1) for n in (5, 9, 3, 12, 7, 2, 30, 4, 6, 8)]
    batches = list(P.packed_iterate_batches(data, 2, 16, seed=3))
    assert "truncated" in capsys.readouterr().out            # the 30-token sequence
    assert len(batches) >= 1
    for b, sid, sst, mask in batches:
        assert b.shape == (2, 17) and b.dtype == torch.int32
        assert sid.shape == sst.shape == mask.shape == (2, 16)
        assert sid.dtype == sst.dtype == torch.int32 and mask.dtype == torch.bool
    again = list(P.packed_iterate_batches(data, 2, 16, seed=3))
    assert all(torch.equal(x, y) for a, b in zip(batches, again) for x, y in zip(a, b))
    assert len(list(P.packed_iterate_batches(data, 2, 16, seed=3, comm_group=_Group(1)))) == len(batches)
    with pytest.raises(PackingError, match="distributed"):
        next(P.packed_iterate_batches(data, 2, 16, comm_group=_Group(2)))
    with pytest.raises(PackingError, match="max_position_embeddings"):
        next(P.packed_iterate_batches(data, 2, 64, max_position_embeddings=32))
    with pytest.raises(PackingError, match="fewer than batch_size"):
        next(P.packed_iterate_batches(data[:2], 8, 64))
    with pytest.raises(PackingError):
        P.pack_indices([], 8, seed=0, epoch=0)
    with pytest.raises(PackingError):
        P.pack_indices([3, 0], 8, seed=0, epoch=0)
    with pytest.raises(PackingError):
        P.pack_indices([3], 0, seed=0, epoch=0)
    it = P.packed_iterate_batches(data, 2, 16, loop=True, seed=3)
    first_epoch = [next(it) for _ in range(len(batches))]
    nxt = next(it)                                            # second epoch reshuffles
    assert nxt[0].shape == (2, 17) and len(first_epoch) == len(batches)
