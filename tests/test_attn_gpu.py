"""GPU parity of flash attention (forward O/L, backward dQ/dK/dV) against the CPU oracle,
through the C ABI.

Tolerances follow the reference's classes (tests/test_attention_kernel_fwd.py:459-466,
tests/test_attention_kernel_bwd.py:345,654,1034,1312) with inputs ~N(0,1):
  fp32 : O 2e-5, L 2e-5, dQ/dK/dV max|diff|/max|ref| 1e-4
  bf16 : O 1.2e-2, L 2e-5 * (1 + |L|), gradients max|diff|/max|ref| 2e-2 (P, dS rounded to bf16)
"""
import pytest
import torch

from mlx_train_perf_b200 import configs
from mlx_train_perf_b200.attention import api as A
from mlx_train_perf_b200.attention.api import flash_attention, flash_attention_with_lse
from mlx_train_perf_b200.attention.segments import PackedMask
from mlx_train_perf_b200.core.loss import check_device_status, device_status
from oracle import attention as oa

from _worst import note

pytestmark = pytest.mark.gpu


def _run(dev, s, hq, hkv, d, dtype, impl, lengths=None, b=1, seed=0):
    inp = configs.attention(s, b=b, hq=hq, hkv=hkv, d=d, dtype=dtype, seed=seed)
    seg_id = seg_start = None
    if lengths is not None:
        seg_id, seg_start = oa.segments_from_lengths(lengths, s)
        seg_id, seg_start = seg_id.expand(b, -1).contiguous(), seg_start.expand(b, -1).contiguous()
    # fp32 kernels are checked against an fp64 evaluation of the oracle, so the host BLAS's own
    # fp32 rounding (which differs between CPUs) stays out of the comparison
    odt = torch.float64 if dtype == torch.float32 else torch.float32
    o_ref, l_ref = oa.flash_attention_reference(inp.q, inp.k, inp.v, scale=inp.scale, seg_id=seg_id, dtype=odt)
    o_saved = o_ref.to(dtype)
    dq_r, dk_r, dv_r = oa.flash_attention_backward(inp.q, inp.k, inp.v, o_saved, l_ref, inp.d_o, scale=inp.scale,
                                                   seg_id=seg_id, dtype=odt)
    o_ref, l_ref, dq_r, dk_r, dv_r = (x.float() for x in (o_ref, l_ref, dq_r, dk_r, dv_r))
    q, k, v = (x.to(dev).requires_grad_(True) for x in (inp.q, inp.k, inp.v))
    pm = None if seg_id is None else PackedMask(seg_id=seg_id.to(dev), seg_start=seg_start.to(dev))
    before = A.VJP_CALLS.get("flash_attention", 0)
    o, lse = flash_attention_with_lse(q, k, v, scale=inp.scale, impl=impl, segments=pm)
    (o.float() * inp.d_o.to(dev).float()).sum().backward()
    torch.cuda.synchronize()
    check_device_status()
    assert A.VJP_CALLS["flash_attention"] == before + 1
    got = (o.float().cpu(), lse.cpu(), q.grad.float().cpu(), k.grad.float().cpu(), v.grad.float().cpu())
    return got, (o_ref, l_ref, dq_r, dk_r, dv_r)


def _check(got, ref, bf16):
    o, l, dq, dk, dv = got
    o_r, l_r, dq_r, dk_r, dv_r = ref
    kind = "bf16" if bf16 else "fp32"
    o_tol = 1.2e-2 if bf16 else 2e-5
    err = note(f"attention {kind} |O - oracle|", (o - o_r).abs().max().item(), o_tol)
    assert err < o_tol, ("O", err)
    err = note(f"attention {kind} |L - oracle| / (1 + |L|)", ((l - l_r).abs() / (1 + l_r.abs())).max().item(), 2e-5)
    assert err < 2e-5, ("L", err)
    tol = 2e-2 if bf16 else 1e-4
    for name, x, y in (("dQ", dq, dq_r), ("dK", dk, dk_r), ("dV", dv, dv_r)):
        rel = note(f"attention {kind} {name} max|diff| / max|oracle|", (x - y).abs().max().item() / y.abs().max().item(), tol)
        assert rel < tol, (name, rel)


@pytest.mark.parametrize(("s", "hq", "hkv", "d"), [(64, 4, 2, 64), (200, 4, 1, 96), (300, 4, 4, 128), (33, 2, 1, 128)])
def test_fp32_simt_causal(cuda_device, s, hq, hkv, d):
    _check(*_run(cuda_device, s, hq, hkv, d, torch.float32, "auto"), bf16=False)


def test_fp32_simt_packed(cuda_device):
    _check(*_run(cuda_device, 250, 4, 2, 64, torch.float32, "auto", lengths=[7, 100, 1, 142]), bf16=False)


@pytest.mark.parametrize(("s", "hq", "hkv"), [(128, 4, 2), (256, 4, 1), (384, 8, 2), (1000, 4, 2), (77, 2, 2)])
def test_bf16_tc_causal(cuda_device, s, hq, hkv):
    # "tc2" forces the two-tile forward (small grids would otherwise take the single-tile one)
    _check(*_run(cuda_device, s, hq, hkv, 128, torch.bfloat16, "tc2"), bf16=True)


@pytest.mark.parametrize(("s", "hq", "hkv", "lengths"), [(384, 4, 2, None), (900, 2, 2, None), (640, 3, 3, [100, 300, 57, 1, 182]),
                                                        (1000, 6, 2, [130, 3, 3, 380, 484])])
def test_bf16_tc_forward_variants(cuda_device, s, hq, hkv, lengths):
    """Odd GQA groups / MHA take the two-query-block pairing of the two-tile forward ("tc2" forces that
    kernel); "tc1" is the single-tile forward kernel; "tc" picks between them by grid size.  All must
    agree with the oracle."""
    for impl in ("tc2", "tc1", "tc"):
        _check(*_run(cuda_device, s, hq, hkv, 128, torch.bfloat16, impl, lengths=lengths), bf16=True)


@pytest.mark.parametrize(("s", "hq", "hkv", "lengths", "b"), [(128, 2, 1, None, 1), (1000, 4, 2, None, 2), (1300, 8, 2, None, 1),
                                                             (640, 4, 1, [100, 300, 57, 1, 182], 1),
                                                             (1000, 2, 1, [130, 3, 3, 380, 484], 2)])
def test_bf16_tc_forward_split_over_keys(cuda_device, s, hq, hkv, lengths, b):
    """"tc2s": every query block's key range split over two CTAs (fp32 partial O, running max and sum per
    row) plus the combine pass -- what a grid of few heads gets by itself.  Shares can be empty (one key
    block) or fully masked for a row (a packed segment that starts in the second share): against the
    oracle, and L against the unsplit kernel."""
    got, ref = _run(cuda_device, s, hq, hkv, 128, torch.bfloat16, "tc2s", lengths=lengths, b=b)
    _check(got, ref, bf16=True)
    plain, _ = _run(cuda_device, s, hq, hkv, 128, torch.bfloat16, "tc2", lengths=lengths, b=b)
    assert (got[1] - plain[1]).abs().max().item() < 5e-6
    assert (got[0] - plain[0]).abs().max().item() <= 2 ** -6   # O: one bf16 ulp at |O| < 4


@pytest.mark.parametrize("impl", ["tc2s", "tc2s3", "tc2s4"])
def test_split_forward_is_reproducible(cuda_device, impl):
    """A forward split over keys adds its shares in index order in the combine pass: O and L must come out
    bit for bit the same on every run, also while another stream keeps the memory system busy, for two,
    three and four shares (some of them empty), and match the unsplit kernel within rounding."""
    dev = cuda_device
    inp = configs.attention(1500, hq=4, hkv=2, d=128, seed=9)
    q, k, v = (x.to(dev) for x in (inp.q, inp.k, inp.v))
    o0, l0 = A.flash_fwd_raw(q, k, v, scale=inp.scale, impl=impl)
    plain_o, plain_l = A.flash_fwd_raw(q, k, v, scale=inp.scale, impl="tc2")
    torch.cuda.synchronize()
    assert (l0 - plain_l).abs().max().item() < 5e-6
    assert (o0.float() - plain_o.float()).abs().max().item() <= 2 ** -6
    side = torch.cuda.Stream()
    junk = torch.empty(64 << 20, dtype=torch.uint8, device=dev)
    for i in range(8):
        if i % 2:
            with torch.cuda.stream(side):
                for _ in range(4):
                    junk.add_(1)
        o, l = A.flash_fwd_raw(q, k, v, scale=inp.scale, impl=impl)
        torch.cuda.synchronize()
        assert torch.equal(o, o0) and torch.equal(l, l0), i
    check_device_status()


@pytest.mark.parametrize(("s", "hq", "hkv", "d", "lengths"), [(300, 4, 2, 64, None), (200, 4, 1, 96, None),
                                                            (520, 4, 2, 64, [130, 3, 380, 7]), (257, 2, 2, 96, [57, 200]),
                                                            (700, 3, 3, 96, None), (1100, 8, 2, 64, [500, 600])])
def test_bf16_head_dim_64_96(cuda_device, s, hq, hkv, d, lengths):
    """bf16 head_dim 64 / 96 have tensor-core kernels of their own (every forward / backward variant), and
    the CUDA-core kernels on request; all against the oracle, the two families against each other, and no
    padded copy of q / k / v is allocated on the way."""
    dev = cuda_device
    b = _run(dev, s, hq, hkv, d, torch.bfloat16, "simt", lengths=lengths)
    _check(*b, bf16=True)

    def peak_of(dd, impl):
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats(dev)
        base = torch.cuda.memory_allocated(dev)
        out = _run(dev, s, hq, hkv, dd, torch.bfloat16, impl, lengths=lengths)
        return out, torch.cuda.max_memory_allocated(dev) - base

    _, peak128 = peak_of(128, "tc")
    for impl in ("tc", "tc1", "tc2", "tc2s", "tcp", "tcg"):
        if impl == "tc2s" and (hq // hkv) % 2 != 0:
            continue                      # the split over keys pairs two q heads of a GQA group
        a, peak = peak_of(d, impl)
        _check(*a, bf16=True)
        assert a[0][0].shape[-1] == d and a[0][2].shape[-1] == d
        assert (a[0][1] - b[0][1]).abs().max().item() < 2e-4          # L of the two kernel families
        if impl == "tc":
            # every tensor of the step scales with head_dim (bar the row statistics and the fp32 partials of small grids,
            # whose rows keep the 128-column pitch): a run that padded q / k / v
            # to 128 would peak where the head_dim-128 run does
            assert peak < (d / 128 + 0.3) * peak128 and peak < 0.95 * peak128, (peak, peak128)


@pytest.mark.parametrize("d", [64, 96])
def test_head_dim_64_96_cost_less_than_128(cuda_device, d):
    """The narrower instantiations issue fewer MMA steps (contractions over head_dim) and narrower MMAs
    (products that are head_dim wide): at S=4096, 32 q / 8 kv heads a forward+backward must take less time
    than at head_dim 128 (on zero-padded copies it took the head_dim-128 time plus seven copies).  Not
    proportionally less: the softmax / elementwise passes, whose work does not depend on head_dim, bound
    these kernels together with the tensor pipe (measured 0.85x at 64, 0.96x at 96)."""
    dev = cuda_device

    def step_ms(dd):
        inp = configs.attention(4096, hq=32, hkv=8, d=dd, seed=0, device=dev)
        def step():
            o, lse = A.flash_fwd_raw(inp.q, inp.k, inp.v, scale=inp.scale)
            A.flash_bwd_raw(inp.q, inp.k, inp.v, o, lse, inp.d_o, scale=inp.scale)
        for _ in range(5):
            step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(30):
            step()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 30

    t128, td = step_ms(128), step_ms(d)
    check_device_status()
    assert td < (0.93 if d == 64 else 1.0) * t128, (d, td, t128)


def test_bf16_tc_batch(cuda_device):
    _check(*_run(cuda_device, 300, 4, 2, 128, torch.bfloat16, "tc2", b=2), bf16=True)
    _check(*_run(cuda_device, 300, 4, 2, 128, torch.bfloat16, "tc1", b=2), bf16=True)


@pytest.mark.parametrize("lengths", [[128, 128, 256], [100, 300, 57, 1, 310], [700], [130, 3, 3, 380, 8]])
def test_bf16_tc_packed(cuda_device, lengths):
    s = sum(lengths)
    _check(*_run(cuda_device, s, 4, 2, 128, torch.bfloat16, "tc2", lengths=lengths), bf16=True)
    _check(*_run(cuda_device, s, 4, 2, 128, torch.bfloat16, "tc", lengths=lengths), bf16=True)


def test_bf16_simt_equals_tc(cuda_device):
    """Two kernels, one truth."""
    a, _ = _run(cuda_device, 300, 4, 2, 128, torch.bfloat16, "tc", lengths=[120, 180])
    b, _ = _run(cuda_device, 300, 4, 2, 128, torch.bfloat16, "simt", lengths=[120, 180])
    # both outputs are rounded to bf16 separately: allow two ulps at |O| < 4 (2 * 2^-6)
    assert (a[0] - b[0]).abs().max().item() <= 2 * 2 ** -6
    assert (a[1] - b[1]).abs().max().item() < 2e-4
    for x, y in zip(a[2:], b[2:]):
        assert (x - y).abs().max().item() / y.abs().max().item() < 2e-2


def test_packed_equals_per_segment_runs(cuda_device):
    """Composition (tests/test_attention_segments.py:32-131): the packed kernel equals the
    causal kernel run on each segment alone."""
    dev = cuda_device
    lengths = [200, 184]
    inp = configs.attention(384, hq=4, hkv=2, d=128, seed=3)
    seg_id, seg_start = oa.segments_from_lengths(lengths)
    q, k, v = inp.q.to(dev), inp.k.to(dev), inp.v.to(dev)
    o_p, l_p = flash_attention_with_lse(q, k, v, scale=inp.scale,
                                        segments=PackedMask(seg_id=seg_id.to(dev), seg_start=seg_start.to(dev)))
    a = 0
    for n in lengths:
        o_s, l_s = flash_attention_with_lse(q[:, :, a:a + n].contiguous(), k[:, :, a:a + n].contiguous(),
                                            v[:, :, a:a + n].contiguous(), scale=inp.scale)
        assert (o_p[:, :, a:a + n].float() - o_s.float()).abs().max().item() < 1.2e-2
        assert (l_p[:, :, a:a + n] - l_s).abs().max().item() < 2e-4
        a += n
    check_device_status()


def test_strided_bshd_views(cuda_device):
    """(B, S, H, d) projections viewed as (B, H, S, d): no transpose copy is needed."""
    dev = cuda_device
    inp = configs.attention(256, hq=4, hkv=2, d=128, seed=4)
    q = inp.q.transpose(1, 2).contiguous().to(dev).transpose(1, 2)
    k = inp.k.transpose(1, 2).contiguous().to(dev).transpose(1, 2)
    v = inp.v.transpose(1, 2).contiguous().to(dev).transpose(1, 2)
    assert not q.is_contiguous()
    o = flash_attention(q, k, v, scale=inp.scale)
    o_ref = oa.math_attention(inp.q, inp.k, inp.v, scale=inp.scale)
    torch.cuda.synchronize()
    check_device_status()
    assert (o.float().cpu() - o_ref).abs().max().item() < 1.2e-2


def test_expanded_kv_heads_get_summed_gradients(cuda_device):
    """k / v expanded over the head axis (stride 0: every q head reads the same storage): the
    operator must copy such aliasing views, or the backward's per-head dK / dV rows would race on one
    buffer.  Autograd then sums the copies' gradients, as for any expand."""
    dev = cuda_device
    inp = configs.attention(200, hq=4, hkv=1, d=128, seed=6)
    k1 = inp.k.to(dev).requires_grad_(True)
    v1 = inp.v.to(dev).requires_grad_(True)
    q = inp.q.to(dev).requires_grad_(True)
    o = flash_attention(q, k1.expand(1, 4, 200, 128), v1.expand(1, 4, 200, 128), scale=inp.scale)   # MHA over copies
    (o.float() * inp.d_o.to(dev).float()).sum().backward()
    torch.cuda.synchronize()
    check_device_status()
    o_ref, l_ref = oa.flash_attention_reference(inp.q, inp.k, inp.v, scale=inp.scale)
    dq_r, dk_r, dv_r = oa.flash_attention_backward(inp.q, inp.k, inp.v, o_ref.to(torch.bfloat16), l_ref, inp.d_o,
                                                   scale=inp.scale)
    assert (o.float().cpu() - o_ref).abs().max().item() < 1.2e-2
    for name, got, ref in (("dQ", q.grad, dq_r), ("dK", k1.grad, dk_r), ("dV", v1.grad, dv_r)):
        rel = (got.float().cpu() - ref).abs().max().item() / ref.abs().max().item()
        assert rel < 2e-2, (name, rel)


def test_validate_segments_refuses_a_broken_mask(cuda_device):
    from mlx_train_perf_b200.errors import AttentionInputError
    dev = cuda_device
    inp = configs.attention(128, hq=2, hkv=1, d=128, seed=7)
    q, k, v = (x.to(dev) for x in (inp.q, inp.k, inp.v))
    seg_id = torch.zeros(1, 128, dtype=torch.int32, device=dev)
    seg_id[0, 64:] = 2                                      # skips id 1
    seg_start = torch.where(seg_id == 0, 0, 64).to(torch.int32)
    with pytest.raises(AttentionInputError, match="PackedMask contract"):
        flash_attention(q, k, v, scale=inp.scale, segments=PackedMask(seg_id=seg_id, seg_start=seg_start),
                        validate_segments=True)


def test_first_row_and_gqa_identities(cuda_device):
    """tests/test_attention_reference.py:95-136 and tests/test_attention_kernel_fwd.py:524-545 on
    the kernels: row 0 returns V[kv,0]; L[0] = scale q0.k0; constant V per kv head shows the
    contiguous h // group mapping."""
    dev = cuda_device
    hq, hkv, s, d = 8, 2, 130, 128
    inp = configs.attention(s, hq=hq, hkv=hkv, d=d, seed=9)
    v = torch.stack([torch.full((s, d), float(j + 1)) for j in range(hkv)])[None].to(torch.bfloat16)
    o, lse = flash_attention_with_lse(inp.q.to(dev), inp.k.to(dev), v.to(dev), scale=inp.scale)
    torch.cuda.synchronize()
    for h in range(hq):
        assert torch.allclose(o[0, h].float().cpu(), torch.full((s, d), float(h // (hq // hkv) + 1)), atol=2e-2)
        want = inp.scale * float(inp.q[0, h, 0].float() @ inp.k[0, h // (hq // hkv), 0].float())
        assert abs(lse[0, h, 0].item() - want) < 1e-4
    check_device_status()


def test_bitwise_repeatable(cuda_device):
    dev = cuda_device
    inp = configs.attention(512, hq=4, hkv=2, d=128, seed=5)
    outs = []
    for _ in range(2):
        q, k, v = (x.to(dev).requires_grad_(True) for x in (inp.q, inp.k, inp.v))
        o = flash_attention(q, k, v, scale=inp.scale)
        (o.float() * inp.d_o.to(dev).float()).sum().backward()
        outs.append((o.clone(), q.grad.clone(), k.grad.clone(), v.grad.clone()))
    torch.cuda.synchronize()
    for a, b in zip(*outs):
        assert torch.equal(a, b)


def test_forward_kernels_agree_on_a_batched_ragged_shape(cuda_device):
    """B=3, S=4100 (ragged last block), 6q/2kv: the two-tile and the single-tile forward agree to one
    bf16 ulp, and sampled rows match a direct fp32 softmax on the device."""
    from mlx_train_perf_b200.attention.api import flash_bwd_raw, flash_fwd_raw
    dev = cuda_device
    b, s, hq, hkv = 3, 4100, 6, 2
    inp = configs.attention(s, b=b, hq=hq, hkv=hkv, d=128, seed=1, device=dev)
    o2, l2 = flash_fwd_raw(inp.q, inp.k, inp.v, scale=inp.scale, impl="tc2")
    o1, l1 = flash_fwd_raw(inp.q, inp.k, inp.v, scale=inp.scale, impl="tc1")
    dq, dk, dv = flash_bwd_raw(inp.q, inp.k, inp.v, o2, l2, inp.d_o, scale=inp.scale)
    torch.cuda.synchronize()
    check_device_status()
    assert (o2.float() - o1.float()).abs().max().item() <= 2 ** -7
    assert (l2 - l1).abs().max().item() < 1e-5
    assert all(torch.isfinite(t.float()).all().item() for t in (dq, dk, dv))
    h, kvh, bi = hq - 1, (hq - 1) // (hq // hkv), b - 1
    rows = torch.tensor([0, 1, 127, 128, s // 2, s - 1], device=dev)
    sc = inp.q[bi, h, rows].float() @ inp.k[bi, kvh].float().T * inp.scale
    sc = sc.masked_fill(torch.arange(s, device=dev)[None, :] > rows[:, None], float("-inf"))
    assert (l2[bi, h, rows] - torch.logsumexp(sc, -1)).abs().max().item() < 2e-5
    assert (o2[bi, h, rows].float() - torch.softmax(sc, -1) @ inp.v[bi, kvh].float()).abs().max().item() < 1.2e-2


def test_forward_workspace_contract(cuda_device):
    """b200tp_flash_fwd_ws through ctypes: the workspace query is 0 for a grid that fills the SMs and
    for shapes that cannot split, non-zero for one kv-head group of a long sequence; a misaligned
    workspace is refused before any launch; without a workspace the forced split runs unsplit and
    gives the two-tile kernel's result bit for bit."""
    import ctypes as C

    from mlx_train_perf_b200 import _lib
    from mlx_train_perf_b200.attention.api import _attn_args, flash_fwd_raw, flash_fwd_workspace_bytes
    dev = cuda_device
    big = configs.attention(256, b=1, hq=4, hkv=1, d=128, seed=3, device=dev)
    assert flash_fwd_workspace_bytes(big.q, big.k, big.v, scale=big.scale) == 0                 # short sequence
    assert flash_fwd_workspace_bytes(big.q, big.k, big.v, scale=big.scale, impl="tc1") == 0
    need = flash_fwd_workspace_bytes(big.q, big.k, big.v, scale=big.scale, impl="tc2s")
    assert need >= 2 * 4 * 256 * (128 + 2) * 4
    q_long = torch.empty(1, 4, 8192, 128, dtype=torch.bfloat16, device=dev)
    k_long = torch.empty(1, 1, 8192, 128, dtype=torch.bfloat16, device=dev)
    assert flash_fwd_workspace_bytes(q_long, k_long, k_long, scale=big.scale) > 0                # splits by itself
    q_many = torch.empty(1, 32, 8192, 128, dtype=torch.bfloat16, device=dev)
    k_many = torch.empty(1, 8, 8192, 128, dtype=torch.bfloat16, device=dev)
    assert flash_fwd_workspace_bytes(q_many, k_many, k_many, scale=big.scale) == 0               # grid fills the SMs

    lib = _lib.load()
    o = torch.empty_like(big.q)
    lse = torch.empty(1, 4, 256, dtype=torch.float32, device=dev)
    a = _attn_args(big.q, big.k, big.v, o, scale=big.scale, segments=None, impl="tc2s")
    ws = torch.empty(need + 256, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    status = device_status(dev).data_ptr()
    rc = lib.b200tp_flash_fwd_ws(C.byref(a), big.q.data_ptr(), big.k.data_ptr(), big.v.data_ptr(), o.data_ptr(),
                                 lse.data_ptr(), ws.data_ptr() + 1, need, stream, status)
    assert rc == _lib.ERR_WORKSPACE
    rc = lib.b200tp_flash_fwd_ws(C.byref(a), big.q.data_ptr(), big.k.data_ptr(), big.v.data_ptr(), o.data_ptr(),
                                 lse.data_ptr(), None, 0, stream, status)
    assert rc == 0
    o2, lse2 = flash_fwd_raw(big.q, big.k, big.v, scale=big.scale, impl="tc2")
    torch.cuda.synchronize()
    check_device_status()
    assert torch.equal(o, o2) and torch.equal(lse, lse2)


@pytest.mark.parametrize(("s", "hq", "hkv", "lengths", "b"), [(300, 4, 2, None, 1), (1000, 8, 2, None, 2), (257, 6, 2, None, 1),
                                                             (640, 4, 1, [100, 300, 57, 1, 182], 1)])
def test_bf16_tc_dkv_group_per_cta(cuda_device, s, hq, hkv, lengths, b):
    """dK / dV with one CTA per (kv head, key block) that walks all q heads of the GQA group ("tcg": what
    a grid of at least two such CTAs per SM gets by itself) against the oracle, and against the
    per-q-head CTAs with fp32 partials and the reduce pass ("tcp"): same sums in another order."""
    got, ref = _run(cuda_device, s, hq, hkv, 128, torch.bfloat16, "tcg", lengths=lengths, b=b)
    _check(got, ref, bf16=True)
    other, _ = _run(cuda_device, s, hq, hkv, 128, torch.bfloat16, "tcp", lengths=lengths, b=b)
    assert torch.equal(got[2], other[2])                                     # dQ does not depend on it
    for x, y in ((got[3], other[3]), (got[4], other[4])):
        assert (x - y).abs().max().item() <= 2 ** -6 * max(1.0, y.abs().max().item())


@pytest.mark.parametrize(("s", "hq", "hkv", "d", "lengths"), [(1000, 4, 2, 128, None), (700, 4, 1, 96, [100, 300, 300]),
                                                              (300, 2, 2, 64, None)])
def test_backward_parts_match_the_whole_backward(cuda_device, s, hq, hkv, d, lengths):
    """`parts="dq"` / `"dkv"` (what the benchmark times one kernel with) give the whole backward's results:
    dQ bit for bit (same kernel, same inputs), dK / dV within rounding of the statistics -- alone, the
    dK / dV kernel takes them from the stand-alone pre-pass instead of the dQ kernel's prologue, which sums
    dO * O in another order."""
    dev = cuda_device
    inp = configs.attention(s, hq=hq, hkv=hkv, d=d, seed=4)
    q, k, v, d_o = (x.to(dev) for x in (inp.q, inp.k, inp.v, inp.d_o))
    pm = None
    if lengths is not None:
        seg_id, seg_start = oa.segments_from_lengths(lengths, s)
        pm = PackedMask(seg_id=seg_id.to(dev), seg_start=seg_start.to(dev))
    o, lse = A.flash_fwd_raw(q, k, v, scale=inp.scale, segments=pm, impl="tc")
    dq, dk, dv = A.flash_bwd_raw(q, k, v, o, lse, d_o, scale=inp.scale, segments=pm, impl="tc")
    dq1, _, _ = A.flash_bwd_raw(q, k, v, o, lse, d_o, scale=inp.scale, segments=pm, impl="tc", parts="dq")
    _, dk2, dv2 = A.flash_bwd_raw(q, k, v, o, lse, d_o, scale=inp.scale, segments=pm, impl="tc", parts="dkv")
    torch.cuda.synchronize()
    check_device_status()
    assert torch.equal(dq1, dq)
    for name, x, y in (("dK", dk2, dk), ("dV", dv2, dv)):
        rel = (x.float() - y.float()).abs().max().item() / y.float().abs().max().item()
        assert rel < 4e-3, (name, rel)      # half a bf16 ulp of the largest element, at most
