"""GPU parity of the fused linear cross-entropy against the CPU oracle, through the C ABI.

Tolerances (max-abs unless noted) follow the reference's classes with head-room for the larger shapes
used here (the end-of-run summary prints the worst error observed per class):
  forward nll / lse / tgt : 1e-5 for fp32 and for bf16 inputs with fp32 accumulation
                            (tests/test_kernel_parity.py:35-44 pins 4e-6 / 5e-6 at N <= 257; worst seen
                            here 4.8e-6 at V up to 40000);
  int4 forward            : same, against dequantise-in-fp32-then-round-to-bf16 weights
                            (the rounding contract stated in tests/test_kernel_quant_parity.py:54-64);
  d_hidden                : max|diff| / max|ref| <= 2e-5 fp32, 1e-2 bf16 on the dense parity cases (worst
                            seen 2.6e-6 / 4.8e-3), 1.5e-2 bf16 elsewhere
                            (tests/test_kernel_backward_parity.py:85,154 pins 2e-6 / 5e-3 abs at
                            weight scale 0.05; g is rounded to bf16 before the second GEMM).
"""
import pytest
import torch

from mlx_train_perf_b200 import configs
from mlx_train_perf_b200.core import loss as L
from mlx_train_perf_b200.core.loss import DenseHead, QuantizedHead, fused_linear_ce, linear_cross_entropy
from oracle import linear_ce as oc

from _worst import note

pytestmark = pytest.mark.gpu

FWD_TOL = 1e-5


def _plant_boundary_targets(t, v, tile=256):
    """Targets at 0, V-1 and tile edges (tests/test_kernel_parity.py:9-44 plants the same)."""
    picks = [0, v - 1, tile - 1, tile, min(v - 1, 2 * tile - 1)]
    for i, p in enumerate(picks):
        if i < t.numel() and p < v:
            t[i] = p
    return t


def _run_dense(dev, n, d, v, dtype, impl, ignore_frac=0.05, seed=0):
    inp = configs.ce_dense(n, d, v, dtype=dtype, ignore_frac=ignore_frac, seed=seed)
    _plant_boundary_targets(inp.targets, v)
    inp.targets[-1] = configs.IGNORE_INDEX
    g = torch.Generator().manual_seed(seed + 100)
    # non-uniform cotangent: alternating sign, varying magnitude
    ct = (torch.rand(n, generator=g) + 0.5) * torch.where(torch.arange(n) % 2 == 0, 1.0, -1.0) / n
    # fp32 kernels are checked against an fp64 evaluation of the oracle (host BLAS rounding differs
    # between CPUs); bf16 kernels against the fp32 one on the bf16-rounded inputs
    odt = torch.float64 if dtype == torch.float32 else torch.float32
    ref_nll, ref_lse, ref_tgt = oc.naive_linear_ce(inp.hidden, inp.weight, inp.targets, dtype=odt)
    ref_dh, _ = oc.chunked_backward(inp.hidden, inp.weight, inp.targets, ref_lse, ct, chunk_size=4096, dtype=odt)
    ref_nll, ref_lse, ref_tgt, ref_dh = (x.float() for x in (ref_nll, ref_lse, ref_tgt, ref_dh))

    h = inp.hidden.to(dev).requires_grad_(True)
    head = DenseHead(weight=inp.weight.to(dev))
    before = dict(L.VJP_CALLS)
    nll, lse, tgt = fused_linear_ce(h, head, inp.targets.to(dev), impl=impl)
    (nll * ct.to(dev)).sum().backward()
    torch.cuda.synchronize()
    L.check_device_status()
    assert L.VJP_CALLS.get("dense", 0) == before.get("dense", 0) + 1
    return (nll.cpu(), lse.cpu(), tgt.cpu(), h.grad.float().cpu()), (ref_nll, ref_lse, ref_tgt, ref_dh), inp


def _check(got, ref, inp, dh_rel):
    nll, lse, tgt, dh = got
    rn, rl, rt, rdh = ref
    kind = "fp32" if dh_rel < 1e-3 else "bf16"
    for name, x, y in (("lse", lse, rl), ("tgt", tgt, rt), ("nll", nll, rn)):
        err = note(f"linear-CE {kind} forward |{name} - oracle|", (x - y).abs().max().item(), FWD_TOL)
        assert err < FWD_TOL, (name, err)
    ign = inp.targets == configs.IGNORE_INDEX
    assert ign.any() and (nll[ign] == 0).all() and (dh[ign] == 0).all()
    rel = note(f"linear-CE {kind} d_hidden max|diff| / max|oracle|", (dh - rdh).abs().max().item() / rdh.abs().max().item(),
               dh_rel)
    assert rel < dh_rel, ("d_hidden rel-to-max", rel)


# (n, d, v): tails on every axis -- n % 128, d % 64, v % 256 all non-zero in the odd cases
SHAPES = [(128, 64, 256), (300, 200, 1000), (257, 328, 4099), (64, 1024, 2048)]


@pytest.mark.parametrize(("n", "d", "v"), SHAPES)
def test_dense_fp32_simt(cuda_device, n, d, v):
    got, ref, inp = _run_dense(cuda_device, n, d, v, torch.float32, "auto")
    _check(got, ref, inp, 2e-5)


@pytest.mark.parametrize(("n", "d", "v"), SHAPES + [(1000, 512, 20000)])
def test_dense_bf16_tc(cuda_device, n, d, v):
    got, ref, inp = _run_dense(cuda_device, n, d, v, torch.bfloat16, "tc")
    _check(got, ref, inp, 1e-2)


def _run_trainable(dev, n, d, v, dtype, impl, seed=7):
    """Trainable dense head: d_hidden and d_weight = g^T @ hidden (core/chunked.py:84-90)."""
    inp = configs.ce_dense(n, d, v, dtype=dtype, ignore_frac=0.05, seed=seed)
    _plant_boundary_targets(inp.targets, v)
    g = torch.Generator().manual_seed(seed + 100)
    ct = (torch.rand(n, generator=g) + 0.5) * torch.where(torch.arange(n) % 2 == 0, 1.0, -1.0) / n
    odt = torch.float64 if dtype == torch.float32 else torch.float32
    _, ref_lse, _ = oc.naive_linear_ce(inp.hidden, inp.weight, inp.targets, dtype=odt)
    ref_dh, ref_dw = oc.chunked_backward(inp.hidden, inp.weight, inp.targets, ref_lse, ct, chunk_size=4096,
                                         want_dw=True, dtype=odt,
                                         round_g_to=torch.bfloat16 if dtype == torch.bfloat16 else None)
    h = inp.hidden.to(dev).requires_grad_(True)
    w = inp.weight.to(dev).requires_grad_(True)
    before = dict(L.VJP_CALLS)
    nll, _, _ = fused_linear_ce(h, DenseHead(weight=w), inp.targets.to(dev), impl=impl)
    (nll * ct.to(dev)).sum().backward()
    torch.cuda.synchronize()
    L.check_device_status()
    assert L.VJP_CALLS.get("dense_trainable", 0) == before.get("dense_trainable", 0) + 1
    assert w.grad is not None and w.grad.dtype == dtype and w.grad.shape == w.shape
    return h.grad.float().cpu(), w.grad.float().cpu(), ref_dh.float(), ref_dw.float()


@pytest.mark.parametrize(("n", "d", "v"), [(128, 64, 256), (300, 200, 1000), (257, 328, 4099)])
def test_trainable_head_fp32(cuda_device, n, d, v):
    dh, dw, rdh, rdw = _run_trainable(cuda_device, n, d, v, torch.float32, "auto")
    assert (dh - rdh).abs().max().item() / rdh.abs().max().item() < 1e-4
    assert (dw - rdw).abs().max().item() / rdw.abs().max().item() < 1e-4


@pytest.mark.parametrize(("n", "d", "v"), [(128, 64, 256), (300, 200, 1000), (257, 328, 4099), (1000, 512, 40000)])
@pytest.mark.parametrize("impl", ["tc", "simt"])
def test_trainable_head_bf16(cuda_device, n, d, v, impl):
    """d_weight in bf16: one rounding of an fp32 sum over the rows -> half a bf16 ulp of the largest
    entry, plus the accumulation-order noise of g's bf16 rounding."""
    if impl == "simt" and v > 5000:
        pytest.skip("the CUDA-core path is covered at the smaller shapes")
    dh, dw, rdh, rdw = _run_trainable(cuda_device, n, d, v, torch.bfloat16, impl)
    assert (dh - rdh).abs().max().item() / rdh.abs().max().item() < 1.5e-2
    assert (dw - rdw).abs().max().item() / rdw.abs().max().item() < 1.5e-2


def test_frozen_dense_head_takes_the_plain_backward(cuda_device):
    """trainable=True but a weight that does not require grad: no d_weight work is done."""
    inp = configs.ce_dense(64, 64, 512, dtype=torch.bfloat16, seed=1)
    h = inp.hidden.to(cuda_device).requires_grad_(True)
    before = dict(L.VJP_CALLS)
    linear_cross_entropy(h, DenseHead(weight=inp.weight.to(cuda_device)), inp.targets.to(cuda_device)).backward()
    assert L.VJP_CALLS.get("dense", 0) == before.get("dense", 0) + 1
    assert L.VJP_CALLS.get("dense_trainable", 0) == before.get("dense_trainable", 0)


def test_two_kernels_one_truth(cuda_device):
    """tcgen05 and CUDA-core kernels on the same bf16 inputs (the reference's MMA-vs-scalar
    cross-check, tests/test_kernel_backward_parity.py:158-191)."""
    a, _, _ = _run_dense(cuda_device, 300, 264, 3000, torch.bfloat16, "tc")
    b, _, _ = _run_dense(cuda_device, 300, 264, 3000, torch.bfloat16, "simt")
    for x, y in zip(a[:3], b[:3]):
        assert (x - y).abs().max().item() < FWD_TOL
    assert (a[3] - b[3]).abs().max().item() / b[3].abs().max().item() < 1.5e-2


def test_multi_chunk_backward_bf16(cuda_device):
    """V beyond one backward chunk (16384 rows) exercises the chunked fp32 accumulation of d_hidden."""
    got, ref, inp = _run_dense(cuda_device, 256, 256, 40000, torch.bfloat16, "tc", seed=3)
    _check(got, ref, inp, 1e-2)


def test_config1_fp32_full(cuda_device):
    """The reference's CPU-runnable benchmark case at full size: N=2048, D=1024, V=32768, fp32, 5 % ignored, upstream
    gradient 1/num_valid.  Loss within 2e-3 relative (the stated contract) and much tighter."""
    inp = configs.ce_dense(2048, 1024, 32768, dtype=torch.float32, ignore_frac=0.05, seed=0)
    ref_nll, ref_lse, ref_tgt = oc.streamed_lse_and_target(inp.hidden, inp.weight, inp.targets)
    ref_dh, _ = oc.chunked_backward(inp.hidden, inp.weight, inp.targets, ref_lse, inp.cotangent)
    dev = cuda_device
    h = inp.hidden.to(dev).requires_grad_(True)
    loss = linear_cross_entropy(h, DenseHead(weight=inp.weight.to(dev)), inp.targets.to(dev), reduction="mean")
    loss.backward()
    torch.cuda.synchronize()
    L.check_device_status()
    ref_loss = ref_nll.sum().item() / inp.num_valid
    assert abs(loss.item() - ref_loss) / ref_loss < 1e-5
    rel = (h.grad.cpu() - ref_dh).abs().max().item() / ref_dh.abs().max().item()
    assert rel < 1e-4, rel


@pytest.mark.parametrize("impl", ["tc", "simt"])
def test_quantized_head(cuda_device, impl):
    n, d, v = 200, 256, 3000
    inp = configs.ce_quant(n, d, v, ignore_frac=0.05, seed=1)
    w_ref = oc.dequantize_int4(inp.w_q, inp.scales, inp.biases, out_dtype=torch.bfloat16)
    ref_nll, ref_lse, ref_tgt = oc.naive_linear_ce(inp.hidden, w_ref, inp.targets)
    ref_dh, _ = oc.chunked_backward(inp.hidden, w_ref, inp.targets, ref_lse, inp.cotangent)
    dev = cuda_device
    head = QuantizedHead(w_q=inp.w_q.to(dev), scales=inp.scales.to(dev), biases=inp.biases.to(dev))
    h = inp.hidden.to(dev).requires_grad_(True)
    nll, lse, tgt = fused_linear_ce(h, head, inp.targets.to(dev), impl=impl)
    (nll * inp.cotangent.to(dev)).sum().backward()
    torch.cuda.synchronize()
    L.check_device_status()
    assert (lse.cpu() - ref_lse).abs().max().item() < FWD_TOL
    assert (nll.cpu() - ref_nll).abs().max().item() < FWD_TOL
    rel = (h.grad.float().cpu() - ref_dh).abs().max().item() / ref_dh.abs().max().item()
    assert rel < 1.5e-2, rel


def test_dequant_matches_oracle_bitwise(cuda_device):
    import ctypes as C
    from mlx_train_perf_b200 import _lib
    inp = configs.ce_quant(4, 512, 777, seed=5)
    ref = oc.dequantize_int4(inp.w_q, inp.scales, inp.biases, out_dtype=torch.bfloat16)
    dev = cuda_device
    wq, sc, bi = inp.w_q.to(dev), inp.scales.to(dev), inp.biases.to(dev)
    out = torch.empty(777, 512, dtype=torch.bfloat16, device=dev)
    rc = _lib.load().b200tp_dequant_int4(wq.data_ptr(), sc.data_ptr(), bi.data_ptr(), _lib.BF16, 0, 777, 512, 64,
                                         out.data_ptr(), _lib.BF16, torch.cuda.current_stream().cuda_stream)
    _lib.check(rc)
    torch.cuda.synchronize()
    assert torch.equal(out.cpu(), ref)


@pytest.mark.parametrize("impl", ["tc", "simt"])
def test_vocab_shards_combine(cuda_device, impl):
    """Vocab-sharded partial triples + combine == unsharded result; partial d_hidden sums; the
    shards' d_weight blocks are the row blocks of the unsharded d_weight."""
    import ctypes as C
    from mlx_train_perf_b200 import _lib
    n, d, v, shards = 260, 128, 3001, 3
    inp = configs.ce_dense(n, d, v, dtype=torch.bfloat16, ignore_frac=0.05, seed=2)
    ref_nll, ref_lse, ref_tgt = oc.naive_linear_ce(inp.hidden, inp.weight, inp.targets)
    ref_dh, ref_dw = oc.chunked_backward(inp.hidden, inp.weight, inp.targets, ref_lse, inp.cotangent, want_dw=True,
                                         round_g_to=torch.bfloat16)
    dev = cuda_device
    h, t = inp.hidden.to(dev), inp.targets.to(dev)
    bounds = [0, 1000, 2000, v]
    parts = torch.empty(shards, 3, n, dtype=torch.float32, device=dev)
    for r in range(shards):
        w = inp.weight[bounds[r]:bounds[r + 1]].contiguous().to(dev)
        m, s, tg, _, _ = L.ce_forward_raw(h, DenseHead(weight=w), t, v_offset=bounds[r], impl=impl, want_lse=False)
        parts[r, 0], parts[r, 1], parts[r, 2] = m, s, tg
    out = torch.empty(3, n, dtype=torch.float32, device=dev)
    rc = _lib.load().b200tp_linear_ce_combine(parts.data_ptr(), shards, n, t.data_ptr(), configs.IGNORE_INDEX,
                                              out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr(),
                                              torch.cuda.current_stream().cuda_stream)
    _lib.check(rc)
    lse, nll, tgt = out[0], out[1], out[2]
    dh = torch.zeros(n, d, dtype=torch.float32, device=dev)
    dws = []
    for r in range(shards):
        w = inp.weight[bounds[r]:bounds[r + 1]].contiguous().to(dev)
        dws.append(torch.empty_like(w))
        L.ce_backward_raw(h, DenseHead(weight=w), t, lse, inp.cotangent.to(dev), v_offset=bounds[r], impl=impl,
                          out_dtype=torch.float32, out=dh, accumulate=True, d_weight=dws[-1])
    torch.cuda.synchronize()
    L.check_device_status()
    assert (lse.cpu() - ref_lse).abs().max().item() < FWD_TOL
    assert (nll.cpu() - ref_nll).abs().max().item() < FWD_TOL
    assert (tgt.cpu() - ref_tgt).abs().max().item() < FWD_TOL
    rel = (dh.cpu() - ref_dh).abs().max().item() / ref_dh.abs().max().item()
    assert rel < 1.5e-2, rel
    dw = torch.cat(dws, dim=0).float().cpu()
    rel = (dw - ref_dw).abs().max().item() / ref_dw.abs().max().item()
    assert rel < 1.5e-2, rel


def test_reductions_and_3d_input(cuda_device):
    dev = cuda_device
    inp = configs.ce_dense(96, 64, 500, dtype=torch.float32, ignore_frac=0.1, seed=4)
    ref_nll, _, _ = oc.naive_linear_ce(inp.hidden, inp.weight, inp.targets)
    head = DenseHead(weight=inp.weight.to(dev))
    h3 = inp.hidden.to(dev).reshape(4, 24, 64)
    t3 = inp.targets.to(dev).reshape(4, 24)
    none = linear_cross_entropy(h3, head, t3, reduction="none")
    assert none.shape == (4, 24)
    assert (none.reshape(-1).cpu() - ref_nll).abs().max().item() < FWD_TOL
    s = linear_cross_entropy(h3, head, t3, reduction="sum").item()
    m = linear_cross_entropy(h3, head, t3, reduction="mean").item()
    assert abs(s - ref_nll.sum().item()) < 1e-3
    assert abs(m - ref_nll.sum().item() / inp.num_valid) < 1e-5


def test_bitwise_repeatable(cuda_device):
    """No atomics anywhere on the path: two runs agree bit for bit (the race tripwire)."""
    dev = cuda_device
    inp = configs.ce_dense(300, 256, 5000, dtype=torch.bfloat16, seed=6)
    head = DenseHead(weight=inp.weight.to(dev))
    outs = []
    for _ in range(2):
        h = inp.hidden.to(dev).requires_grad_(True)
        nll, lse, tgt = fused_linear_ce(h, head, inp.targets.to(dev))
        (nll * inp.cotangent.to(dev)).sum().backward()
        outs.append((nll.clone(), lse.clone(), h.grad.clone()))
    torch.cuda.synchronize()
    for a, b in zip(*outs):
        assert torch.equal(a, b)


def _dequant_on_gpu(dev, w_q, scales, biases, d):
    """The standalone dequantisation kernel (bit-exact against the oracle, see above)."""
    from mlx_train_perf_b200 import _lib
    v = w_q.shape[0]
    out = torch.empty(v, d, dtype=torch.bfloat16, device=dev)
    qdt = _lib.BF16 if scales.dtype == torch.bfloat16 else _lib.F32
    rc = _lib.load().b200tp_dequant_int4(w_q.data_ptr(), scales.data_ptr(), biases.data_ptr(), qdt, 0, v, d, 64,
                                         out.data_ptr(), _lib.BF16, torch.cuda.current_stream().cuda_stream)
    _lib.check(rc)
    return out


@pytest.mark.parametrize("case", ["typical", "degenerate", "fp32_params"])
def test_inkernel_dequant_is_bit_identical_to_dequant_then_dense(cuda_device, case):
    """The tensor-core kernels expand a 4-bit head inside their pipeline (two packed bf16 instructions
    per code pair, or fp32 fma for groups where that could round differently).  Contract: the bits of
    `b200tp_dequant_int4` -- so the quantized head must give EXACTLY the lse / nll / d_hidden of the
    dense kernels run on that kernel's output, including on scale / bias pairs chosen to sit on the
    fast path's boundary (tiny or zero biases, zero scales, biases far above the scale)."""
    dev = cuda_device
    n, d, v = 200, 320, 3000          # v % 256 != 0, d % 256 != 0: partial tiles on both operands' axes
    inp = configs.ce_quant(n, d, v, ignore_frac=0.05, seed=11)
    sc, bi = inp.scales.clone(), inp.biases.clone()
    if case == "degenerate":
        g = torch.Generator().manual_seed(3)
        kind = torch.randint(0, 6, sc.shape, generator=g)
        sf, bf = sc.float(), bi.float()
        bf = torch.where(kind == 0, torch.zeros_like(bf), bf)                    # zero bias
        bf = torch.where(kind == 1, sf * 2.0 ** -9, bf)                          # bias just inside the fast path
        bf = torch.where(kind == 2, sf * 2.0 ** -10 * 1.5, bf)                   # just outside: fp32 path
        bf = torch.where(kind == 3, sf * 2.0 ** -20, bf)                         # far outside
        bf = torch.where(kind == 4, sf * 2.0 ** 18, bf)                          # bias dwarfs the code term
        sf = torch.where(kind == 5, torch.zeros_like(sf), sf)                    # zero scale
        sc, bi = sf.to(torch.bfloat16), bf.to(torch.bfloat16)
    if case == "fp32_params":
        g = torch.Generator().manual_seed(4)
        sc = (torch.randn(sc.shape, generator=g) * 0.01).abs()
        bi = -8.0 * sc + torch.randn(sc.shape, generator=g) * 1e-4
    wq, sc, bi = inp.w_q.to(dev), sc.to(dev), bi.to(dev)
    w_dense = _dequant_on_gpu(dev, wq, sc, bi, d)
    h, t, ct = inp.hidden.to(dev), inp.targets.to(dev), inp.cotangent.to(dev)
    qhead, dhead = QuantizedHead(w_q=wq, scales=sc, biases=bi), DenseHead(weight=w_dense)
    outs = []
    for head, impl in ((qhead, "tc_inline"), (dhead, "tc"), (qhead, "tc_chunked")):
        _, _, tgt, lse, nll = L.ce_forward_raw(h, head, t, impl=impl)
        dh = L.ce_backward_raw(h, head, t, lse, ct, impl=impl)
        outs.append((lse, nll, tgt, dh))
    torch.cuda.synchronize()
    L.check_device_status()
    for other in (1, 2):
        for name, a, b in zip(("lse", "nll", "tgt", "d_hidden"), outs[0], outs[other]):
            assert torch.equal(a, b), (case, other, name, (a.float() - b.float()).abs().max().item())
    # and the whole thing still agrees with the oracle
    w_ref = oc.dequantize_int4(inp.w_q, sc.cpu(), bi.cpu(), out_dtype=torch.bfloat16)
    if case == "fp32_params":
        # fp32 scales: scale * code is no longer exact, so the kernel's single fma rounding and the oracle's
        # separate multiply and add may differ in the last fp32 bit, i.e. (rarely) by one bf16 ulp
        diff = (w_dense.cpu().float() - w_ref.float()).abs()
        assert (diff <= w_ref.float().abs() * 2.0 ** -7).all() and (diff > 0).float().mean().item() < 1e-3
    else:
        assert torch.equal(w_dense.cpu(), w_ref)
    ref_nll, ref_lse, _ = oc.naive_linear_ce(inp.hidden, w_ref, inp.targets)
    scale = 1.0 + ref_lse.abs().max().item()
    assert (outs[0][0].cpu() - ref_lse).abs().max().item() < FWD_TOL * scale


@pytest.mark.parametrize("impl", ["tc_inline", "tc_chunked"])
def test_quantized_head_multi_chunk_and_workspace(cuda_device, impl):
    """V beyond one backward chunk, both dequantisation forms; with the head expanded inside the kernels
    the workspaces hold no dequantised weights."""
    import ctypes as C
    from mlx_train_perf_b200 import _lib
    dev = cuda_device
    n, d, v = 256, 256, 40000
    inp = configs.ce_quant(n, d, v, ignore_frac=0.05, seed=12)
    w_ref = oc.dequantize_int4(inp.w_q, inp.scales, inp.biases, out_dtype=torch.bfloat16)
    ref_nll, ref_lse, _ = oc.naive_linear_ce(inp.hidden, w_ref, inp.targets)
    ref_dh, _ = oc.chunked_backward(inp.hidden, w_ref, inp.targets, ref_lse, inp.cotangent)
    head = QuantizedHead(w_q=inp.w_q.to(dev), scales=inp.scales.to(dev), biases=inp.biases.to(dev))
    h, t = inp.hidden.to(dev), inp.targets.to(dev)
    _, _, _, lse, nll = L.ce_forward_raw(h, head, t, impl=impl)
    dh = L.ce_backward_raw(h, head, t, lse, inp.cotangent.to(dev), impl=impl)
    torch.cuda.synchronize()
    L.check_device_status()
    assert (lse.cpu() - ref_lse).abs().max().item() < FWD_TOL
    assert (nll.cpu() - ref_nll).abs().max().item() < FWD_TOL
    rel = (dh.float().cpu() - ref_dh).abs().max().item() / ref_dh.abs().max().item()
    assert rel < 1.5e-2, rel
    a, _keep = L._ce_args(h, head, t, v_offset=0, ignore_index=configs.IGNORE_INDEX, impl=impl)
    lib = _lib.load()
    fwd = lib.b200tp_linear_ce_fwd_workspace_bytes(C.byref(a))
    bwd = lib.b200tp_linear_ce_bwd_workspace_bytes(C.byref(a), _lib.BF16)
    w_chunk = 13568 * d * 2                                                # ceil(40000 / 3) vocab rows, padded to 256
    if impl == "tc_inline":
        assert fwd < w_chunk // 4, fwd                                        # partial triples only
        assert bwd <= n * 16384 * 2 + n * d * 4 + 1024, bwd                    # g chunk + fp32 accumulator, no W chunk
    else:
        assert w_chunk <= fwd < w_chunk + (1 << 20), fwd
        assert bwd >= n * 13568 * 2 + w_chunk, bwd


@pytest.mark.parametrize("quant", [False, True])
def test_staged_backward_is_the_plain_backward(cuda_device, quant):
    """`b200tp_linear_ce_bwd_stage` issues the same launches as the plain backward, the last chunk's
    d_hidden GEMM in slabs of whole waves: the fp32 partial must come out bit for bit the same, and
    the rows reported done after each stage must already hold their final values."""
    import ctypes as C
    from mlx_train_perf_b200 import _lib
    dev = cuda_device
    n, d, v = 5000, 1024, 20000        # 40 row blocks x 4 column tiles = 160 tiles > 148 CTAs; two vocab chunks
    if quant:
        inp = configs.ce_quant(n, d, v, ignore_frac=0.05, seed=13)
        head = QuantizedHead(w_q=inp.w_q.to(dev), scales=inp.scales.to(dev), biases=inp.biases.to(dev))
    else:
        inp = configs.ce_dense(n, d, v, dtype=torch.bfloat16, ignore_frac=0.05, seed=13)
        head = DenseHead(weight=inp.weight.to(dev))
    h, t, ct = inp.hidden.to(dev), inp.targets.to(dev), inp.cotangent.to(dev)
    impl = "tc_inline" if quant else "tc"      # the in-kernel expansion at a shape with 40 row blocks
    _, _, _, lse, _ = L.ce_forward_raw(h, head, t, impl=impl)
    plain = L.ce_backward_raw(h, head, t, lse, ct, out_dtype=torch.float32, impl=impl)
    lib = _lib.load()
    a, _keep = L._ce_args(h, head, t, v_offset=0, ignore_index=configs.IGNORE_INDEX, impl=impl)
    nbytes = lib.b200tp_linear_ce_bwd_workspace_bytes(C.byref(a), _lib.F32)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    stages = 2
    out = torch.full((n, d), float("nan"), dtype=torch.float32, device=dev)
    done = C.c_int64(0)
    seen = []
    for s in range(stages):
        rc = lib.b200tp_linear_ce_bwd_stage(C.byref(a), lse.data_ptr(), ct.data_ptr(), out.data_ptr(), _lib.F32, 0,
                                            stages, s, C.byref(done), ws.data_ptr(), nbytes,
                                            torch.cuda.current_stream().cuda_stream, L.device_status(dev).data_ptr())
        _lib.check(rc)
        torch.cuda.synchronize()
        r = int(done.value)
        seen.append(r)
        assert torch.equal(out[:r], plain[:r]), (s, r)
    L.check_device_status()
    assert seen[-1] == n and 0 < seen[0] < n and seen[0] % 128 == 0, seen
    assert torch.equal(out, plain)


def test_backward_chunk_bound_option(cuda_device):
    """`reserved` lowers the vocab rows per backward chunk (less scratch, more launches); only the
    fp32 accumulation order over chunks changes."""
    import ctypes as C
    from mlx_train_perf_b200 import _lib
    dev = cuda_device
    inp = configs.ce_dense(300, 256, 9000, dtype=torch.bfloat16, ignore_frac=0.05, seed=14)
    h, t, ct = inp.hidden.to(dev), inp.targets.to(dev), inp.cotangent.to(dev)
    head = DenseHead(weight=inp.weight.to(dev))
    _, _, _, lse, _ = L.ce_forward_raw(h, head, t)
    ref = L.ce_backward_raw(h, head, t, lse, ct)
    lib = _lib.load()
    a, _keep = L._ce_args(h, head, t, v_offset=0, ignore_index=configs.IGNORE_INDEX, impl="tc")
    big = lib.b200tp_linear_ce_bwd_workspace_bytes(C.byref(a), _lib.BF16)
    a.reserved = 8                                                           # chunks of at most 2048 vocab rows
    small = lib.b200tp_linear_ce_bwd_workspace_bytes(C.byref(a), _lib.BF16)
    assert small < big
    ws = torch.empty(small, dtype=torch.uint8, device=dev)
    out = torch.empty_like(h)
    rc = lib.b200tp_linear_ce_bwd(C.byref(a), lse.data_ptr(), ct.data_ptr(), out.data_ptr(), _lib.BF16, 0,
                                  ws.data_ptr(), small, torch.cuda.current_stream().cuda_stream,
                                  L.device_status(dev).data_ptr())
    _lib.check(rc)
    torch.cuda.synchronize()
    L.check_device_status()
    rel = (out.float() - ref.float()).abs().max().item() / ref.float().abs().max().item()
    assert rel < 1e-2, rel


def test_inkernel_dequant_repeatable_under_load(cuda_device):
    """Forty row blocks, two vocab chunks, scales / biases at an address that forces the one-load-per-stage
    parameter path (the dequantising warps then lag the tensor pipe, the case in which a code slot handed
    back too early was once overwritten under a slow warp): six runs of the in-kernel backward must equal the
    chunked one bit for bit."""
    dev = cuda_device
    n, d, v = 5000, 1024, 20000
    inp = configs.ce_quant(n, d, v, ignore_frac=0.05, seed=13)
    wq, sc, bi = inp.w_q.to(dev), inp.scales.to(dev), inp.biases.to(dev)
    h, t, ct = inp.hidden.to(dev), inp.targets.to(dev), inp.cotangent.to(dev)

    def misaligned(x):
        buf = torch.empty(x.numel() + 8, dtype=x.dtype, device=dev)
        view = buf[1:1 + x.numel()].view_as(x)
        view.copy_(x)
        return view

    for scales, biases in ((sc, bi), (misaligned(sc), misaligned(bi))):
        head = QuantizedHead(w_q=wq, scales=scales, biases=biases)
        _, _, _, lse, _ = L.ce_forward_raw(h, head, t, impl="tc_chunked")
        ref = L.ce_backward_raw(h, head, t, lse, ct, impl="tc_chunked", out_dtype=torch.float32)
        lse_first = None
        for _ in range(6):
            _, _, _, lse_i, _ = L.ce_forward_raw(h, head, t, impl="tc_inline")
            got = L.ce_backward_raw(h, head, t, lse, ct, impl="tc_inline", out_dtype=torch.float32)
            # the two forwards split the vocabulary differently (per chunk / over the whole shard), so their
            # lse agree to rounding; the in-kernel one must repeat itself exactly
            lse_first = lse_i if lse_first is None else lse_first
            assert torch.equal(lse_i, lse_first) and (lse_i - lse).abs().max().item() < FWD_TOL
            assert torch.equal(got, ref)
    torch.cuda.synchronize()
    L.check_device_status()


@pytest.mark.parametrize("reduction", ["mean", "sum"])
@pytest.mark.parametrize("trainable", [False, True])
def test_reduced_loss_is_formed_in_the_library(cuda_device, reduction, trainable):
    """`mean` / `sum` run one small reduce kernel after the row combine and one small cotangent kernel
    before the backward: same loss and gradients as reducing the per-row losses with torch, the count
    of supervised rows comes back with the loss, and no torch reduction kernel is launched."""
    from mlx_train_perf_b200.core.loss import reduced_linear_cross_entropy
    dev = cuda_device
    inp = configs.ce_dense(700, 256, 5000, dtype=torch.bfloat16, ignore_frac=0.2, seed=21)
    t = inp.targets.to(dev)

    def run(fused):
        h = inp.hidden.to(dev).requires_grad_(True)
        w = inp.weight.to(dev).requires_grad_(trainable)
        head = DenseHead(weight=w, trainable=trainable)
        if fused:
            loss, count = reduced_linear_cross_entropy(h, head, t, reduction=reduction)
            assert int(count.item()) == inp.num_valid
        else:
            nll = linear_cross_entropy(h, head, t, reduction="none", validate_targets=False)
            loss = nll.sum() / (inp.num_valid if reduction == "mean" else 1)
        (loss * 3.0).backward()
        return loss.detach(), h.grad, (w.grad if trainable else None)

    names = []
    try:
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            fused = run(True)
            torch.cuda.synchronize()
        names = [e.key for e in prof.key_averages()]
    except Exception:       # no CUPTI on this host: the numerical checks below still run
        fused = run(True)
    plain = run(False)
    torch.cuda.synchronize()
    L.check_device_status()
    assert abs(fused[0].item() - plain[0].item()) <= 2e-6 * max(1.0, abs(plain[0].item()))
    rel = (fused[1].float() - plain[1].float()).abs().max().item() / plain[1].float().abs().max().item()
    assert rel < 1e-2, rel      # the cotangent reaches the kernels through one rounding less
    if trainable:
        rel = (fused[2].float() - plain[2].float()).abs().max().item() / plain[2].float().abs().max().item()
        assert rel < 1e-2, rel
    if names:
        assert any("loss_reduce_kernel" in n for n in names) and any("loss_cotangent_kernel" in n for n in names), names
        assert not any("reduce_kernel" in n and "loss_reduce_kernel" not in n and "dkv" not in n for n in names), names


@pytest.mark.parametrize("mean", [True, False])
def test_masked_loss_of_existing_rows(cuda_device, mean):
    """`masked_loss` (what a vocab-sharded caller runs on its replicated per-row losses): sum / mean over
    the supervised rows, their count, and the cotangent vector of the backward, against torch."""
    dev = cuda_device
    g = torch.Generator().manual_seed(3)
    n = 5000
    nll = torch.rand(n, generator=g) * 9
    t = torch.randint(0, 1000, (n,), generator=g)
    t[torch.rand(n, generator=g) < 0.3] = configs.IGNORE_INDEX
    valid = t != configs.IGNORE_INDEX
    nll[~valid] = 0.0
    up = torch.tensor([2.5])
    loss, count, ct = L.masked_loss(nll.to(dev), t.to(dev), mean=mean, upstream=up.to(dev))
    torch.cuda.synchronize()
    cnt = int(valid.sum())
    ref = nll.double().sum().item() / (cnt if mean else 1)
    assert int(count.item()) == cnt
    assert abs(loss.item() - ref) <= 2e-6 * abs(ref)
    ref_ct = valid.float() * (2.5 / cnt if mean else 2.5)
    assert torch.equal(ct.cpu() == 0, ~valid)
    assert (ct.cpu() - ref_ct).abs().max().item() <= 1e-6 * ref_ct.max().item()
    # all rows ignored: loss 0, count 0, zero cotangent (no division by zero)
    t0 = torch.full((64,), configs.IGNORE_INDEX)
    loss, count, ct = L.masked_loss(torch.zeros(64, device=dev), t0.to(dev), mean=mean)
    assert loss.item() == 0.0 and count.item() == 0.0 and not ct.any()
