"""Parity at the full sizes of the benchmark configurations (bf16 and 4-bit lm_head at N=8192,
V=151936; causal GQA attention at S=2048..16384; the packed 16384-token row), where the oracle cannot materialise the whole
problem: rows of the loss and kv-head groups of attention are independent, so the oracle is run
in full precision on a seeded SUBSET (sampled rows with the full vocabulary; one kv-head group
with its four query heads; packed segments one at a time -- the composition property of
tests/test_attention_segments.py:32-131) and compared with the same slice of the full-size
kernel result.  Contract at these sizes: loss within 2e-3 relative, gradients within bf16
tolerance (fp32 accumulation)."""
import pytest
import torch

from mlx_train_perf_b200 import configs
from mlx_train_perf_b200.attention.api import flash_bwd_raw, flash_fwd_raw
from mlx_train_perf_b200.attention.segments import PackedMask
from mlx_train_perf_b200.core import loss as L
from mlx_train_perf_b200.core.loss import DenseHead, QuantizedHead
from oracle import attention as oa
from oracle import linear_ce as oc
from _worst import note

pytestmark = pytest.mark.gpu


def _sample_rows(n, k, seed):
    g = torch.Generator().manual_seed(seed)
    idx = torch.randperm(n, generator=g)[:k].sort().values
    return idx


def _check_ce_rows(dev, inp, head, w_cpu_for_oracle, rows):
    h, t, ct = inp.hidden.to(dev), inp.targets.to(dev), inp.cotangent.to(dev)
    torch.cuda.reset_peak_memory_stats(dev)
    base = torch.cuda.memory_allocated(dev)
    _, _, tgt, lse, nll = L.ce_forward_raw(h, head, t)
    dh = L.ce_backward_raw(h, head, t, lse, ct)
    torch.cuda.synchronize()
    L.check_device_status()
    extra = torch.cuda.max_memory_allocated(dev) - base
    n, v = h.shape[0], w_cpu_for_oracle.shape[0]
    assert extra < n * v * 2 // 3, f"peak extra memory {extra} is of the order of an (N, V) tensor"
    hs, ts, cs = inp.hidden[rows], inp.targets[rows], inp.cotangent[rows]
    r_nll, r_lse, r_tgt = oc.streamed_lse_and_target(hs, w_cpu_for_oracle, ts, chunk_size=16384)
    r_dh, _ = oc.chunked_backward(hs, w_cpu_for_oracle, ts, r_lse, cs, chunk_size=16384)
    nll_s, lse_s, tgt_s = nll.cpu()[rows], lse.cpu()[rows], tgt.cpu()[rows]
    assert note("full-size linear-CE |lse - oracle| / |lse|", ((lse_s - r_lse).abs() / r_lse.abs()).max().item(), 2e-5) < 2e-5
    scale = 1.0 + r_lse.abs().max().item()          # fp32 resolution grows with the logit magnitude
    assert (tgt_s - r_tgt).abs().max().item() < 1e-5 * scale
    valid = ts != configs.IGNORE_INDEX
    assert note("full-size linear-CE |nll - oracle| / nll (contract 2e-3)",
                ((nll_s - r_nll).abs()[valid] / r_nll[valid]).max().item(), 2e-3) < 2e-3      # the stated contract
    assert (nll_s - r_nll).abs().max().item() < 1e-5 * scale                          # and much tighter
    loss = float((nll.cpu() * inp.cotangent).sum())
    assert 0 < loss < 1e4                                                             # finite masked-mean loss
    rel = note("full-size linear-CE d_hidden max|diff| / max|oracle|",
               (dh.float().cpu()[rows] - r_dh).abs().max().item() / r_dh.abs().max().item(), 1.5e-2)
    assert rel < 1.5e-2, rel
    ign = inp.targets == configs.IGNORE_INDEX
    assert (nll.cpu()[ign] == 0).all() and (dh.cpu()[ign] == 0).all()


def test_config2_bf16_flagship(cuda_device):
    """N=8192, D=4096, V=151936 bf16, 3 % ignored; 24 sampled rows against the oracle."""
    dev = cuda_device
    inp = configs.ce_dense(8192, 4096, 151936, dtype=torch.bfloat16, ignore_frac=0.03, seed=0)
    rows = _sample_rows(8192, 24, 1)
    rows[0] = int((inp.targets == configs.IGNORE_INDEX).nonzero()[0])      # include an ignored row
    _check_ce_rows(dev, inp, DenseHead(weight=inp.weight.to(dev)), inp.weight, rows)


def test_config5_linear_ce_n16384(cuda_device):
    """The packed row of config 5 through the loss: N=16384, D=4096, V=151936 bf16, a quarter of the
    positions unsupervised (pad slots and prompt tokens of a packed row); 16 sampled rows."""
    dev = cuda_device
    inp = configs.ce_dense(16384, 4096, 151936, dtype=torch.bfloat16, ignore_frac=0.25, seed=5)
    rows = _sample_rows(16384, 16, 5)
    rows[0] = int((inp.targets == configs.IGNORE_INDEX).nonzero()[0])
    _check_ce_rows(dev, inp, DenseHead(weight=inp.weight.to(dev)), inp.weight, rows)


def test_config3_int4_head(cuda_device):
    """Same shape with the 4-bit affine group-64 head (codes uniform, scales |N(0,0.01)|, biases -8 scale)."""
    dev = cuda_device
    inp = configs.ce_quant(8192, 4096, 151936, ignore_frac=0.03, seed=0)
    w_ref = oc.dequantize_int4(inp.w_q, inp.scales, inp.biases, out_dtype=torch.bfloat16)
    head = QuantizedHead(w_q=inp.w_q.to(dev), scales=inp.scales.to(dev), biases=inp.biases.to(dev))
    _check_ce_rows(dev, inp, head, w_ref, _sample_rows(8192, 16, 2))


def _attn_group_check(dev, inp, kv_head, seg_lengths=None, one_head_at_a_time=False):
    """Full-size kernel run; oracle on one kv head and its query heads, segment by segment."""
    b, hq, s, d = inp.q.shape
    group = hq // inp.k.shape[1]
    q, k, v, d_o = (x.to(dev) for x in (inp.q, inp.k, inp.v, inp.d_o))
    pm = None
    if seg_lengths is not None:
        pm = PackedMask(seg_id=inp.seg_id.to(dev), seg_start=inp.seg_start.to(dev))
    torch.cuda.reset_peak_memory_stats(dev)
    base = torch.cuda.memory_allocated(dev)
    o, lse = flash_fwd_raw(q, k, v, scale=inp.scale, segments=pm)
    dq, dk, dv = flash_bwd_raw(q, k, v, o, lse, d_o, scale=inp.scale, segments=pm)
    torch.cuda.synchronize()
    L.check_device_status()
    extra = torch.cuda.max_memory_allocated(dev) - base
    # O, dQ, dK, dV, L, the row statistics of the backward as a bf16 operand tile (32 bytes per row) and
    # the fp32 per-q-head dK / dV partials: all O(S), nothing O(S^2)
    linear = 2 * o.numel() * 2 + 2 * dk.numel() * 2 + (1 + 8) * lse.numel() * 4 + 2 * q.numel() * 4
    assert extra <= linear + (1 << 20), f"{extra - linear} bytes beyond the O(S) buffers: an (S, S) buffer?"
    assert linear < hq * s * s * 2 or s < 1024
    hs = slice(kv_head * group, (kv_head + 1) * group)
    bounds, a = [], 0
    for n in (seg_lengths or [s]):
        bounds.append((a, a + n))
        a += n
    o_c, l_c, dq_c, dk_c, dv_c = (x.float().cpu() for x in (o[:, hs], lse[:, hs], dq[:, hs], dk[:, kv_head:kv_head + 1],
                                                              dv[:, kv_head:kv_head + 1]))
    worst = {"O": 0.0, "L": 0.0, "dQ": 0.0, "dK": 0.0, "dV": 0.0}
    def oracle(qs, ks, vs, o_saved, dos):
        if not one_head_at_a_time:
            o_r, l_r = oa.flash_attention_reference(qs, ks, vs, scale=inp.scale)
            return (o_r, l_r) + tuple(oa.flash_attention_backward(qs, ks, vs, o_saved, l_r, dos, scale=inp.scale))
        # heads of a group are independent except for the dK / dV sum over the group
        outs = []
        for h in range(qs.shape[1]):
            sl = slice(h, h + 1)
            o_r, l_r = oa.flash_attention_reference(qs[:, sl], ks, vs, scale=inp.scale)
            outs.append((o_r, l_r) + tuple(oa.flash_attention_backward(qs[:, sl], ks, vs, o_saved[:, sl], l_r,
                                                                        dos[:, sl], scale=inp.scale)))
        o_r, l_r, dq_r = (torch.cat([x[i] for x in outs], dim=1) for i in range(3))
        return o_r, l_r, dq_r, sum(x[3] for x in outs), sum(x[4] for x in outs)

    for lo, hi in bounds:
        qs, ks, vs = inp.q[:, hs, lo:hi], inp.k[:, kv_head:kv_head + 1, lo:hi], inp.v[:, kv_head:kv_head + 1, lo:hi]
        dos = inp.d_o[:, hs, lo:hi]
        o_r, l_r, dq_r, dk_r, dv_r = oracle(qs, ks, vs, o_c[:, :, lo:hi].to(torch.bfloat16), dos)
        worst["O"] = max(worst["O"], (o_c[:, :, lo:hi] - o_r).abs().max().item())
        worst["L"] = max(worst["L"], ((l_c[:, :, lo:hi] - l_r).abs() / (1 + l_r.abs())).max().item())
        for name, got, ref in (("dQ", dq_c[:, :, lo:hi], dq_r), ("dK", dk_c[:, :, lo:hi], dk_r),
                               ("dV", dv_c[:, :, lo:hi], dv_r)):
            worst[name] = max(worst[name], (got - ref).abs().max().item() / ref.abs().max().item())
    note("full-size attention |O - oracle|", worst["O"], 1.2e-2)
    note("full-size attention |L - oracle| / (1 + |L|)", worst["L"], 2e-5)
    for name in ("dQ", "dK", "dV"):
        note(f"full-size attention {name} max|diff| / max|oracle|", worst[name], 2e-2)
    assert worst["O"] < 1.2e-2 and worst["L"] < 2e-5, worst
    assert worst["dQ"] < 2e-2 and worst["dK"] < 2e-2 and worst["dV"] < 2e-2, worst


def test_config4_causal_gqa_s8192(cuda_device):
    """B=1, 32q/8kv heads, S=8192, d=128 bf16; kv head 5 and its query heads 20-23 in full."""
    inp = configs.attention(8192, seed=0)
    _attn_group_check(cuda_device, inp, kv_head=5)


@pytest.mark.parametrize("s", [2048, 4096, 16384])
def test_config4_sweep(cuda_device, s):
    """The other sequence lengths of the sweep; at 16384 the oracle runs the group's query heads one
    at a time (an (S, S) fp32 matrix is 1 GiB there)."""
    inp = configs.attention(s, seed=0)
    _attn_group_check(cuda_device, inp, kv_head=(s // 2048) % 8, one_head_at_a_time=s > 8192)


def test_config5_packed_16384(cuda_device):
    """16384 packed tokens, segment lengths U[128, 4096] (numpy rng 1): packed kernel == oracle run
    on each segment alone, for one kv-head group; fused loss on the same tokens with ignore_index at
    each segment's last token."""
    dev = cuda_device
    att, _ = configs.packed(16384, seed=1, with_ce=False)
    assert sum(att.seg_lengths) == 16384 and all(128 <= n <= 4096 for n in att.seg_lengths[:-1])
    _attn_group_check(dev, att, kv_head=2, seg_lengths=att.seg_lengths)
    ce = configs.ce_dense(16384, 4096, 151936, ignore_frac=0.0, seed=1)
    ends = torch.tensor(att.seg_lengths).cumsum(0) - 1
    ce.targets[ends] = configs.IGNORE_INDEX
    valid = ce.targets != configs.IGNORE_INDEX
    ce.cotangent, ce.num_valid = valid.float() / valid.sum(), int(valid.sum())
    rows = _sample_rows(16384, 12, 3)
    rows[0] = ends[0]
    _check_ce_rows(dev, ce, DenseHead(weight=ce.weight.to(dev)), ce.weight, rows)
