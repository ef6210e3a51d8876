// Self-test of the bounded device-side wait every tensor-core kernel of this library relies on.
//
// One CTA arms an mbarrier that nothing ever completes and waits on it with the same
// `mbar_wait` the kernels use.  The wait gives up after its time limit, the kernel raises the
// CTA's abort flag, records B200TP_DEV_TIMEOUT_OTHER in the caller's status word and returns
// normally: no trap, no fault, the context stays usable.  A second warp shows that an abort
// raised by one role ends the waits of the others promptly.
#include <cuda_runtime.h>

#include "../../include/b200tp.h"
#include "common.h"
#include "ptx.cuh"

namespace b200tp {
namespace {

__global__ void __launch_bounds__(64, 1) bounded_wait_kernel(int* status, unsigned long long* waited_ns) {
  __shared__ uint64_t never;      // armed, never completed
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&never, 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  const unsigned long long t0 = global_timer_ns();
  if (threadIdx.x == 0) {
    // role A: waits until the limit expires, then aborts the CTA
    const bool ok = mbar_wait(&never, 0, &abort_flag);
    if (!ok) {
      atomicExch(&abort_flag, 1);
      if (status != nullptr) atomicCAS(status, 0, static_cast<int>(kDevTimeoutOther));
    }
    if (waited_ns != nullptr) waited_ns[0] = global_timer_ns() - t0;
  } else if (threadIdx.x == 32) {
    // role B: its own wait ends because role A raised the abort flag (or on its own limit)
    mbar_wait(&never, 0, &abort_flag);
    if (waited_ns != nullptr) waited_ns[1] = global_timer_ns() - t0;
  }
}

}  // namespace
}  // namespace b200tp

extern "C" int b200tp_selftest_bounded_wait(unsigned long long* waited_ns, void* stream, int* status) {
  using namespace b200tp;
  if (status == nullptr) return fail(B200TP_ERR_LOSS_INPUT, "status is null");
  int rc = require_sm100();
  if (rc) return rc;
  bounded_wait_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(status, waited_ns);
  B200TP_CUDA_OK(cudaGetLastError());
  return B200TP_OK;
}
