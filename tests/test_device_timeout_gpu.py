"""The bounded device-side wait and its status plumbing, without faulting the GPU.

Every inter-role wait in the tensor-core kernels is the same bounded `mbar_wait`: after its limit
it returns, the kernel records a status word the host reads at its next synchronisation and the CTA
leaves through its normal teardown.  The library's self-test kernel arms a barrier nothing ever
completes; the test lets that wait run out, checks the status, the typed error, how long the two
roles waited, and that the context and the library still work afterwards."""
import pytest
import torch

from mlx_train_perf_b200 import _lib, configs
from mlx_train_perf_b200.core import loss as L
from mlx_train_perf_b200.core.loss import DenseHead, fused_linear_ce
from mlx_train_perf_b200.errors import DeviceTimeoutError

pytestmark = pytest.mark.gpu


def test_wait_runs_out_status_is_raised_and_context_survives(cuda_device):
    dev = cuda_device
    lib = _lib.load()
    status = L.device_status(dev)
    status.zero_()
    waited = torch.zeros(2, dtype=torch.int64, device=dev)
    with torch.cuda.device(dev):
        rc = lib.b200tp_selftest_bounded_wait(waited.data_ptr(), torch.cuda.current_stream(dev).cuda_stream,
                                              status.data_ptr())
    _lib.check(rc)
    torch.cuda.synchronize(dev)
    assert int(status.item()) == 104                       # B200TP_DEV_TIMEOUT_OTHER
    a_ns, b_ns = (int(x) for x in waited.tolist())
    assert 1.9e9 < a_ns < 4e9, a_ns                        # the 2 s limit, not forever
    assert b_ns < a_ns + 5e7, (a_ns, b_ns)                 # the second role left on the first one's abort
    with pytest.raises(DeviceTimeoutError, match="104"):
        L.check_device_status(dev)
    assert int(status.item()) == 0                         # reading the status clears it
    # the context is intact: a normal forward + backward still runs and reports no status
    inp = configs.ce_dense(128, 64, 512, dtype=torch.bfloat16, seed=0)
    h = inp.hidden.to(dev).requires_grad_(True)
    nll, _, _ = fused_linear_ce(h, DenseHead(weight=inp.weight.to(dev)), inp.targets.to(dev))
    nll.sum().backward()
    torch.cuda.synchronize(dev)
    L.check_device_status(dev)
    assert torch.isfinite(h.grad.float()).all()
