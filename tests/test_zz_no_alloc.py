"""The no-allocation forward (`b200tp_linear_ce_fwd_static`) against the regular forward.

Some callers cannot get device memory at all -- the GPU belongs to a framework's pool they
have no handle to, or an allocation's device-wide synchronisation is unaffordable where they
run -- so they cannot supply the workspace `b200tp_linear_ce_fwd` asks for.  The static variant
keeps its partial buffer inside the library.  This file checks, through the C ABI, that it
returns what the regular entry point returns, on two calls in a row that share (and so reuse)
the built-in buffer, and that it refuses shapes beyond that buffer.

Collected last on purpose (file name), so a failure here cannot hide other results of a run
that stops at the first failure.
"""
import ctypes as C

import pytest
import torch

from mlx_train_perf_b200 import _lib, configs
from mlx_train_perf_b200.core import loss as L
from mlx_train_perf_b200.core.loss import DenseHead

pytestmark = pytest.mark.gpu

TOL = 1e-5   # the forward tolerance of tests/test_ce_gpu.py


def _static_forward(hidden, weight, targets, v_offset=0):
    lib = _lib.load()
    dev = hidden.device
    n, d = hidden.shape
    a = _lib.CeArgs()
    a.hidden, a.weight, a.targets = hidden.data_ptr(), weight.data_ptr(), targets.data_ptr()
    a.n, a.d, a.v_local, a.v_offset = n, d, weight.shape[0], v_offset
    a.dtype, a.quant_bits, a.ignore_index, a.impl = _lib.BF16, 0, configs.IGNORE_INDEX, 0
    out = torch.full((5, n), float("nan"), dtype=torch.float32, device=dev)   # outputs only: caller-owned
    rc = lib.b200tp_linear_ce_fwd_static(C.byref(a), out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr(),
                                         out[3].data_ptr(), out[4].data_ptr(),
                                         torch.cuda.current_stream(dev).cuda_stream,
                                         L.device_status(dev).data_ptr())
    return rc, out


def test_static_forward_matches_workspace_forward_twice(cuda_device):
    dev = cuda_device
    # Two different shapes back to back: the second call finds the first call's partials in
    # the shared buffer and must not be affected by them.
    for n, d, v, seed in ((700, 256, 9000, 0), (300, 512, 4099, 1)):
        inp = configs.ce_dense(n, d, v, dtype=torch.bfloat16, ignore_frac=0.05, seed=seed)
        h, w, t = inp.hidden.to(dev), inp.weight.to(dev), inp.targets.to(dev)
        ref = L.ce_forward_buffer(h, DenseHead(weight=w), t, impl="tc")
        rc, out = _static_forward(h, w, t)
        _lib.check(rc)
        torch.cuda.synchronize()
        L.check_device_status()
        assert not torch.isnan(out).any()
        for row, name in enumerate(("row_max", "row_sumexp", "tgt_logit", "lse", "nll")):
            scale = 1.0 + ref[row].abs().max().item() if name == "row_sumexp" else 1.0
            err = (out[row] - ref[row]).abs().max().item()
            assert err <= TOL * scale, (name, err)


def test_static_forward_allocates_no_device_memory(cuda_device):
    """The point of the entry point: between a warm first call and the end of a second one the device's
    free memory does not move (the caller's tensors exist beforehand; the library creates nothing), and
    the result still matches the oracle-tested workspace forward and the oracle itself."""
    from oracle import linear_ce as oc
    dev = cuda_device
    inp = configs.ce_dense(513, 256, 7001, dtype=torch.bfloat16, ignore_frac=0.05, seed=2)
    h, w, t = inp.hidden.to(dev), inp.weight.to(dev), inp.targets.to(dev)
    rc, _ = _static_forward(h, w, t)          # first call on the device: address look-up, function attributes
    _lib.check(rc)
    lib = _lib.load()
    a = _lib.CeArgs()
    a.hidden, a.weight, a.targets = h.data_ptr(), w.data_ptr(), t.data_ptr()
    a.n, a.d, a.v_local, a.v_offset = 513, 256, 7001, 0
    a.dtype, a.quant_bits, a.ignore_index, a.impl = _lib.BF16, 0, configs.IGNORE_INDEX, 0
    out = torch.full((5, 513), float("nan"), dtype=torch.float32, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    status = L.device_status(dev).data_ptr()
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(dev)
    rc = lib.b200tp_linear_ce_fwd_static(C.byref(a), out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr(),
                                         out[3].data_ptr(), out[4].data_ptr(), stream, status)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info(dev)
    _lib.check(rc)
    L.check_device_status()
    assert free_after == free_before, (free_before, free_after)
    ref_nll, ref_lse, _ = oc.naive_linear_ce(inp.hidden, inp.weight, inp.targets)
    assert (out[3].cpu() - ref_lse).abs().max().item() <= TOL
    assert (out[4].cpu() - ref_nll).abs().max().item() <= TOL


def test_static_forward_fit_boundary(cuda_device):
    """Shapes whose partial triples fill the built-in array exactly are served; one row more is refused."""
    dev = cuda_device
    lib = _lib.load()
    limit = 6 << 20
    # a one-tile vocabulary has a single split: 3 x N x 4 bytes of partials
    n_fit = limit // 12
    for n, expect_ok in ((n_fit, True), (n_fit + 1, False)):
        h = torch.zeros(n, 64, dtype=torch.bfloat16, device=dev)
        w = torch.zeros(256, 64, dtype=torch.bfloat16, device=dev)
        t = torch.zeros(n, dtype=torch.int64, device=dev)
        a = _lib.CeArgs()
        a.hidden, a.weight, a.targets = h.data_ptr(), w.data_ptr(), t.data_ptr()
        a.n, a.d, a.v_local, a.dtype, a.ignore_index = n, 64, 256, _lib.BF16, -100
        ws = lib.b200tp_linear_ce_fwd_workspace_bytes(C.byref(a))
        out = torch.empty(5, n, dtype=torch.float32, device=dev)
        rc = lib.b200tp_linear_ce_fwd_static(C.byref(a), out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr(),
                                             out[3].data_ptr(), out[4].data_ptr(),
                                             torch.cuda.current_stream(dev).cuda_stream, L.device_status(dev).data_ptr())
        torch.cuda.synchronize()
        if expect_ok:
            assert ws <= limit + 3 * 256, ws
            _lib.check(rc)
            assert torch.isfinite(out[3]).all()
        else:
            assert rc == _lib.ERR_WORKSPACE
    L.check_device_status()


def test_static_forward_refuses_oversized_and_unsupported(cuda_device):
    dev = cuda_device
    lib = _lib.load()
    h = torch.zeros(8, 64, dtype=torch.bfloat16, device=dev)
    w = torch.zeros(256, 64, dtype=torch.bfloat16, device=dev)
    t = torch.zeros(8, dtype=torch.int64, device=dev)
    a = _lib.CeArgs()
    a.hidden, a.weight, a.targets = h.data_ptr(), w.data_ptr(), t.data_ptr()
    # far more rows than 6 MiB of partial triples can hold; refused before anything is read
    a.n, a.d, a.v_local, a.dtype, a.ignore_index = 1 << 22, 64, 1 << 20, _lib.BF16, -100
    out = torch.zeros(5, 8, dtype=torch.float32, device=dev)
    rc = lib.b200tp_linear_ce_fwd_static(C.byref(a), out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr(),
                                         None, None, torch.cuda.current_stream(dev).cuda_stream, None)
    assert rc == _lib.ERR_WORKSPACE
    assert b"built-in" in lib.b200tp_last_error()
    a.n, a.v_local, a.dtype = 8, 256, _lib.F32
    rc = lib.b200tp_linear_ce_fwd_static(C.byref(a), out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr(),
                                         None, None, torch.cuda.current_stream(dev).cuda_stream, None)
    assert rc == _lib.ERR_UNSUPPORTED_HEAD
    # a CUDA-core request is refused rather than silently served by the tensor-core kernels
    a.dtype, a.impl = _lib.BF16, _lib.IMPL["simt"]
    rc = lib.b200tp_linear_ce_fwd_static(C.byref(a), out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr(),
                                         None, None, torch.cuda.current_stream(dev).cuda_stream, None)
    assert rc == _lib.ERR_UNSUPPORTED_HEAD
