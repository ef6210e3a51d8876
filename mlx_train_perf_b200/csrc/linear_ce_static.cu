// Forward linear cross-entropy for callers that must not allocate device memory.
//
// Who this is for: code that runs where `cudaMalloc` is off the table -- a loss plugin called
// from inside a framework that has already handed the whole GPU to its own memory pool and
// gives the plugin no allocator handle, or a latency-critical training / serving loop that
// cannot afford the device-wide synchronisation an allocation implies.  Such a caller can
// still provide the inputs and the five (N,) output vectors, but has nowhere to get the
// per-split partial buffer the regular forward needs as `workspace`.
//
// Here that buffer is a fixed array in the library's own device image
// (`g_static_scratch`, B200TP_STATIC_SCRATCH_BYTES = 6 MiB).  Every GPU that loads the
// library carries those 6 MiB until the process exits.  The entry point serves dense bf16
// heads on the tensor-core path only and refuses any shape whose partial triples
// (3 x splits x N floats) do not fit.
//
// Sharing: all calls on a device use the same array and it keeps whatever the previous call
// left in it.  Nothing in it has to start at zero -- each (row, split) slot the combine step
// reads is written by the logits kernel of the same call first -- so no clearing pass runs.
// Two calls that overlap on the GPU (different streams, or different threads without
// ordering) would overwrite each other's partials: callers must order them.
//
// The device address of the array is looked up with cudaGetSymbolAddress the first time the
// entry point runs on a device (with that device current) and cached; make that first call
// before starting any stream capture.
#include <mutex>
#include <string>

#include "common.h"
#include "linear_ce_simt.h"
#include "linear_ce_tc.h"

namespace b200tp {
namespace {

constexpr size_t kStaticScratchBytes = 6u << 20;
static_assert(kStaticScratchBytes == B200TP_STATIC_SCRATCH_BYTES, "header and source disagree");

// File-scope device array.  In host code this name is only a handle for the runtime, never
// a device address: the address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

int static_scratch_ptr(float** out) {
  static std::mutex mu;
  static float* cached[64] = {nullptr};
  int dev = 0;
  B200TP_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(B200TP_ERR_CUDA, "device ordinal out of range");
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == nullptr) {
    void* p = nullptr;
    B200TP_CUDA_OK(cudaGetSymbolAddress(&p, g_static_scratch));
    if (p == nullptr) return fail(B200TP_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
    cached[dev] = static_cast<float*>(p);
  }
  *out = cached[dev];
  return B200TP_OK;
}

}  // namespace
}  // namespace b200tp

using namespace b200tp;

extern "C" int b200tp_linear_ce_fwd_static(const b200tp_ce_args* a, float* row_max, float* row_sumexp,
                                           float* tgt_logit, float* lse, float* nll, void* stream_v, int* status) {
  if (a == nullptr) return fail(B200TP_ERR_LOSS_INPUT, "args is null");
  if (a->n <= 0 || a->d <= 0 || a->v_local <= 0 || a->n > (1ll << 30) || a->v_local > (1ll << 30))
    return fail(B200TP_ERR_LOSS_INPUT, "n, d and v_local must be positive and below 2^30");
  if (a->hidden == nullptr || a->weight == nullptr || a->targets == nullptr)
    return fail(B200TP_ERR_LOSS_INPUT, "hidden / weight / targets is null");
  if (row_max == nullptr || row_sumexp == nullptr || tgt_logit == nullptr)
    return fail(B200TP_ERR_LOSS_INPUT, "row_max / row_sumexp / tgt_logit outputs are required");
  if (a->quant_bits != 0 || a->dtype != B200TP_BF16 || a->d % 8 != 0)
    return fail(B200TP_ERR_UNSUPPORTED_HEAD,
                "the no-allocation forward serves dense bf16 heads with a hidden size that is a multiple of 8; "
                "use b200tp_linear_ce_fwd with a workspace for everything else");
  if (a->impl == B200TP_IMPL_SIMT)
    return fail(B200TP_ERR_UNSUPPORTED_HEAD,
                "the no-allocation forward has no CUDA-core variant (impl=simt needs an (N, chunk) fp32 workspace); "
                "use b200tp_linear_ce_fwd");
  int rc = require_sm100();
  if (rc) return rc;
  const int splits = ce_tc_fwd_splits(a->n, a->v_local);
  const size_t need = 3ull * static_cast<size_t>(splits) * static_cast<size_t>(a->n) * sizeof(float);
  if (need > kStaticScratchBytes)
    return fail(B200TP_ERR_WORKSPACE,
                "shape needs " + std::to_string(need) + " bytes of partial triples (3 x " + std::to_string(splits) +
                    " splits x " + std::to_string(a->n) + " rows x 4), more than the built-in " +
                    std::to_string(kStaticScratchBytes) + "-byte scratch; use b200tp_linear_ce_fwd with a workspace");
  float* scratch = nullptr;
  rc = static_scratch_ptr(&scratch);
  if (rc) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  float* pm = scratch;
  float* ps = pm + static_cast<size_t>(splits) * a->n;
  float* pt = ps + static_cast<size_t>(splits) * a->n;
  rc = ce_tc_launch_fwd(a->hidden, a->weight, a->v_local, a->n, a->d, 0, a->v_local, a->v_offset, a->targets,
                        a->ignore_index, splits, pm, ps, pt, nullptr, stream, status);
  if (rc) return rc;
  return launch_combine(pm, ps, pt, a->n, splits, a->n, a->targets, a->ignore_index, row_max, row_sumexp, tgt_logit,
                        lse, nll, stream);
}
