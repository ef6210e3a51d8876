"""The CPU oracle against every literal known-answer test the reference's own suite holds for
the two hot paths (the reference's random-data tests need MLX and cannot be regenerated)."""
import math

import pytest
import torch

from oracle import attention as oa
from oracle import linear_ce as oc


def test_hand_computed_two_rows():
    # tests/test_naive.py:9-18 of the reference: D=2, V=3, logits row0 = [1, 0, -1].
    hidden = torch.tensor([[1.0, 0.0], [0.0, 1.0]])
    w = torch.tensor([[1.0, 0.0], [0.0, 0.0], [-1.0, 0.0]])
    targets = torch.tensor([0, 1])
    nll, lse, tgt = oc.naive_linear_ce(hidden, w, targets)
    lse0 = math.log(math.exp(1.0) + math.exp(0.0) + math.exp(-1.0))
    assert abs(nll[0].item() - (lse0 - 1.0)) < 1e-6
    assert abs(nll[1].item() - math.log(3.0)) < 1e-6
    assert abs(lse[0].item() - lse0) < 1e-6 and abs(tgt[0].item() - 1.0) < 1e-7


def test_matches_torch_cross_entropy():
    # tests/test_naive.py:21-28 (their second oracle is nn.losses.cross_entropy).
    g = torch.Generator().manual_seed(0)
    hidden = torch.randn(32, 16, generator=g)
    w = torch.randn(100, 16, generator=g)
    targets = torch.randint(0, 100, (32,), generator=g)
    ours, _, _ = oc.naive_linear_ce(hidden, w, targets)
    theirs = torch.nn.functional.cross_entropy(hidden @ w.T, targets, reduction="none")
    assert (ours - theirs).abs().max().item() < 1e-5


def test_output_is_fp32_for_bf16_inputs():
    hidden = torch.randn(4, 8).to(torch.bfloat16)
    w = torch.randn(10, 8).to(torch.bfloat16)
    nll, _, _ = oc.naive_linear_ce(hidden, w, torch.tensor([0, 1, 2, 3]))
    assert nll.dtype == torch.float32


def test_int4_layout_low_nibble_first():
    # tests/test_quant_layout.py:5-16: (V, D/8) words, 8 nibbles per word, low nibble first,
    # w = scale * nib + bias.
    g = torch.Generator().manual_seed(17)
    codes = torch.randint(0, 16, (8, 64), generator=g)
    w_q = oc.pack_int4(codes)
    assert tuple(w_q.shape) == (8, 8) and w_q.dtype == torch.int32
    scales = torch.rand(8, 1, generator=g).to(torch.bfloat16)
    biases = (-8 * scales.float()).to(torch.bfloat16)
    w_dq = oc.dequantize_int4(w_q, scales, biases, out_dtype=torch.float32)
    for k in (0, 1, 7, 8, 63):
        packed = int(w_q[0, k // 8].item()) & 0xFFFFFFFF
        nib = (packed >> (4 * (k % 8))) & 0xF
        assert nib == int(codes[0, k])
        manual = float(scales[0, 0]) * nib + float(biases[0, 0])
        assert abs(manual - float(w_dq[0, k])) < 1e-6
    assert torch.equal(oc.unpack_int4(w_q), codes)


def test_streamed_equals_naive_and_chunk_tail():
    g = torch.Generator().manual_seed(1)
    h = torch.randn(37, 24, generator=g)
    w = torch.randn(301, 24, generator=g) * 0.2
    t = torch.randint(0, 301, (37,), generator=g)
    t[3] = oc.IGNORE_INDEX
    t[5], t[6], t[7] = 0, 300, 127   # boundary targets: first, last, chunk edge
    a = oc.naive_linear_ce(h, w, t)
    b = oc.streamed_lse_and_target(h, w, t, chunk_size=128)
    for x, y in zip(a, b):
        assert (x - y).abs().max().item() < 2e-6
    assert a[0][3].item() == 0.0 and a[2][3].item() == 0.0


def test_shard_combine_equals_naive():
    g = torch.Generator().manual_seed(2)
    h = torch.randn(19, 16, generator=g)
    w = torch.randn(200, 16, generator=g)
    t = torch.randint(0, 200, (19,), generator=g)
    t[0] = oc.IGNORE_INDEX
    parts = [oc.shard_partials(h, w[a:b], t, a) for a, b in ((0, 70), (70, 140), (140, 200))]
    nll, lse, tgt = oc.combine_partials([p[0] for p in parts], [p[1] for p in parts], [p[2] for p in parts], t)
    ref = oc.naive_linear_ce(h, w, t)
    for x, y in zip((nll, lse, tgt), ref):
        assert (x - y).abs().max().item() < 2e-6


def test_chunked_backward_matches_autograd():
    g = torch.Generator().manual_seed(3)
    h = torch.randn(21, 12, generator=g, dtype=torch.float64)
    w = torch.randn(90, 12, generator=g, dtype=torch.float64)
    t = torch.randint(0, 90, (21,), generator=g)
    t[4] = oc.IGNORE_INDEX
    ct = torch.randn(21, generator=g, dtype=torch.float64)    # non-uniform cotangent
    hh = h.clone().requires_grad_(True)
    ww = w.clone().requires_grad_(True)
    logits = hh @ ww.T
    valid = t != oc.IGNORE_INDEX
    nll = torch.nn.functional.cross_entropy(logits, torch.where(valid, t, 0), reduction="none") * valid
    (nll * ct).sum().backward()
    _, lse, _ = oc.naive_linear_ce(h, w, t, dtype=torch.float64)
    dh, dw = oc.chunked_backward(h, w, t, lse, ct, chunk_size=32, want_dw=True, dtype=torch.float64)
    assert (dh - hh.grad).abs().max().item() < 1e-10
    assert (dw - ww.grad).abs().max().item() < 1e-10
    assert dh[4].abs().max().item() == 0.0


def test_segment_allowed_literal():
    # tests/test_attention_segments.py:68-87.
    seg_id = torch.tensor([[0, 0, 1, 1]], dtype=torch.int32)
    allowed = oa.segment_allowed(seg_id)
    expected = torch.tensor([[True, False, False, False], [True, True, False, False],
                             [False, False, True, False], [False, False, True, True]])[None, None]
    assert allowed.shape == (1, 1, 4, 4) and allowed.dtype == torch.bool
    assert torch.equal(allowed, expected)


def _rand_qkv(b, hq, hkv, n, d, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(b, hq, n, d, generator=g), torch.randn(b, hkv, n, d, generator=g),
            torch.randn(b, hkv, n, d, generator=g))


def test_causal_first_row_attends_only_itself():
    # tests/test_attention_reference.py:95-108.
    hq, hkv, n, d = 4, 2, 8, 4
    q, k, v = _rand_qkv(1, hq, hkv, n, d, 3)
    o = oa.math_attention(q, k, v, scale=d ** -0.5)
    for h in range(hq):
        assert torch.allclose(o[0, h, 0], v[0, oa.kv_head_for(h, hq // hkv), 0], atol=1e-5)


@pytest.mark.parametrize(("hq", "hkv"), [(4, 2), (8, 2)])
def test_gqa_uses_contiguous_convention(hq, hkv):
    # tests/test_attention_reference.py:111-136: kv head j holds the constant j+1.
    n, d = 4, 8
    q, k, _ = _rand_qkv(1, hq, hkv, n, d, 5)
    v = torch.stack([torch.full((n, d), float(j + 1)) for j in range(hkv)])[None]
    o = oa.math_attention(q, k, v, scale=1.0)
    for h in range(hq):
        assert torch.allclose(o[0, h], torch.full((n, d), float(h // (hq // hkv) + 1)))


def test_lse_row0_is_scaled_q0_k0():
    # tests/test_attention_kernel_fwd.py:524-545: L[0] = scale * q0 . k0.
    q, k, v = _rand_qkv(1, 2, 1, 16, 8, 7)
    _, lse = oa.flash_attention_reference(q, k, v, scale=0.3)
    for h in range(2):
        assert abs(lse[0, h, 0].item() - 0.3 * float(q[0, h, 0] @ k[0, 0, 0])) < 1e-5


def test_backward_matches_autograd_and_segment_composition():
    # tests/test_attention_reference.py:153-202 (gradient anchor) and
    # tests/test_attention_segments.py:90-131 (packed == per-segment runs).
    q, k, v = _rand_qkv(1, 4, 2, 24, 8, 11)
    q, k, v = q.double(), k.double(), v.double()
    g = torch.Generator().manual_seed(12)
    d_o = torch.randn(1, 4, 24, 8, generator=g, dtype=torch.float64)
    scale = 0.35
    seg_id, _ = oa.segments_from_lengths([10, 14])
    for sid in (None, seg_id):
        qq, kk, vv = (x.clone().requires_grad_(True) for x in (q, k, v))
        kg = kk.repeat_interleave(2, dim=1)
        vg = vv.repeat_interleave(2, dim=1)
        s = (qq @ kg.transpose(-1, -2)) * scale
        mask = torch.tril(torch.ones(24, 24, dtype=torch.bool))[None, None]
        if sid is not None:
            mask = oa.segment_allowed(sid)
        o_ref = torch.softmax(s.masked_fill(~mask, -math.inf), dim=-1) @ vg
        (o_ref * d_o).sum().backward()
        o, lse = oa.flash_attention_reference(q, k, v, scale=scale, seg_id=sid, dtype=torch.float64)
        assert (o - o_ref.detach()).abs().max().item() < 1e-12
        dq, dk, dv = oa.flash_attention_backward(q, k, v, o, lse, d_o, scale=scale, seg_id=sid,
                                                 dtype=torch.float64)
        assert (dq - qq.grad).abs().max().item() < 1e-10
        assert (dk - kk.grad).abs().max().item() < 1e-10
        assert (dv - vv.grad).abs().max().item() < 1e-10
    # packed == running each segment alone
    o_p, l_p = oa.flash_attention_reference(q, k, v, scale=scale, seg_id=seg_id, dtype=torch.float64)
    o_a, l_a = oa.flash_attention_reference(q[:, :, :10], k[:, :, :10], v[:, :, :10], scale=scale,
                                            dtype=torch.float64)
    o_b, l_b = oa.flash_attention_reference(q[:, :, 10:], k[:, :, 10:], v[:, :, 10:], scale=scale,
                                            dtype=torch.float64)
    assert torch.allclose(o_p[:, :, :10], o_a, atol=1e-12) and torch.allclose(o_p[:, :, 10:], o_b, atol=1e-12)
    assert torch.allclose(l_p[:, :, :10], l_a, atol=1e-12) and torch.allclose(l_p[:, :, 10:], l_b, atol=1e-12)


def test_zero_padding_the_head_dim_changes_nothing():
    """The identity the head_dim 64 / 96 route of the tensor-core kernels rests on: zero columns
    appended to q, k, v (and dO) leave O, L, dQ, dK, dV unchanged and come back as zero columns."""
    import torch.nn.functional as F
    torch.manual_seed(0)
    b, hq, hkv, s, d = 1, 4, 2, 40, 64
    q, k, v, d_o = (torch.randn(b, h, s, d, dtype=torch.float64) for h in (hq, hkv, hkv, hq))
    pad = lambda t: F.pad(t, (0, 128 - d))
    o, l = oa.flash_attention_reference(q, k, v, scale=d ** -0.5, dtype=torch.float64)
    o_p, l_p = oa.flash_attention_reference(pad(q), pad(k), pad(v), scale=d ** -0.5, dtype=torch.float64)
    assert torch.equal(l, l_p) and torch.equal(o_p[..., :d], o) and (o_p[..., d:] == 0).all()
    g = oa.flash_attention_backward(q, k, v, o, l, d_o, scale=d ** -0.5, dtype=torch.float64)
    g_p = oa.flash_attention_backward(pad(q), pad(k), pad(v), o_p, l_p, pad(d_o), scale=d ** -0.5, dtype=torch.float64)
    for x, x_p in zip(g, g_p):
        assert torch.allclose(x_p[..., :d], x, rtol=0, atol=1e-14) and (x_p[..., d:] == 0).all()
