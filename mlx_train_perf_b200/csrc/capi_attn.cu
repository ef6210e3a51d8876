// C ABI of flash attention: argument checks and dispatch between the tcgen05 and SIMT
// implementations; also the status / version entry points.
#include <string>

#include "common.h"
#include "flash.h"

namespace b200tp {
const char* last_error_cstr();

namespace {

int check_attn(const b200tp_attn_args* a) {
  if (a == nullptr) return fail(B200TP_ERR_ATTN_INPUT, "args is null");
  if (a->b < 1) return fail(B200TP_ERR_ATTN_INPUT, "batch must be >= 1; got " + std::to_string(a->b));
  if (a->hq < 1 || a->hkv < 1 || a->s < 1) return fail(B200TP_ERR_ATTN_INPUT, "heads and sequence length must be >= 1");
  if (a->hq % a->hkv != 0)
    return fail(B200TP_ERR_ATTN_INPUT, "Hq=" + std::to_string(a->hq) + " must be a multiple of Hkv=" +
                                           std::to_string(a->hkv) + " for GQA grouping");
  if (a->dtype != B200TP_F32 && a->dtype != B200TP_BF16)
    return fail(B200TP_ERR_UNSUPPORTED_ATTN, "only fp32 / bf16 tensors are supported");
  if (a->d != 64 && a->d != 96 && a->d != 128)
    return fail(B200TP_ERR_UNSUPPORTED_ATTN, "head_dim must be one of 64, 96, 128 (got " + std::to_string(a->d) + ")");
  if (!a->causal) return fail(B200TP_ERR_UNSUPPORTED_ATTN, "only causal=True is supported");
  if ((a->seg_id == nullptr) != (a->seg_start == nullptr))
    return fail(B200TP_ERR_ATTN_INPUT, "seg_id and seg_start must be given together");
  if (a->impl != B200TP_IMPL_AUTO && a->impl != B200TP_IMPL_TC && a->impl != B200TP_IMPL_SIMT)
    return fail(B200TP_ERR_ATTN_INPUT, "unknown impl selector");
  return B200TP_OK;
}

bool tc_serves(const b200tp_attn_args* a) {
  if (a->dtype != B200TP_BF16) return false;   // head_dim 64 / 96 / 128 (check_attn) all have tensor-core kernels
  const int64_t* strides[4] = {a->q_stride, a->k_stride, a->v_stride, a->o_stride};
  for (auto st : strides)
    for (int i = 0; i < 3; ++i)
      if (st[i] % 8 != 0) return false;  // TMA wants 16-byte strides
  return true;
}

// 1 = tcgen05, 2 = SIMT, negative = refusal
int pick(const b200tp_attn_args* a) {
  if (a->impl == B200TP_IMPL_SIMT) return 2;
  if (a->impl == B200TP_IMPL_TC) {
    if (!tc_serves(a)) {
      fail(B200TP_ERR_UNSUPPORTED_ATTN,
           "the tensor-core path serves bf16 tensors with 16-byte aligned strides; use impl=simt");
      return -1;
    }
    return 1;
  }
  return tc_serves(a) ? 1 : 2;
}

}  // namespace
}  // namespace b200tp

using namespace b200tp;

extern "C" {

const char* b200tp_status_string(int code) {
  switch (code) {
    case B200TP_OK: return "ok";
    case B200TP_ERR_LOSS_INPUT: return "loss input error";
    case B200TP_ERR_UNSUPPORTED_HEAD: return "unsupported head";
    case B200TP_ERR_ATTN_INPUT: return "attention input error";
    case B200TP_ERR_UNSUPPORTED_ATTN: return "unsupported attention configuration";
    case B200TP_ERR_WORKSPACE: return "workspace error";
    case B200TP_ERR_CUDA: return "CUDA error";
    case B200TP_ERR_NO_DEVICE: return "no sm_100 device";
    case B200TP_DEV_TIMEOUT_PRODUCER: return "device wait timed out (TMA producer)";
    case B200TP_DEV_TIMEOUT_MMA: return "device wait timed out (MMA issuer)";
    case B200TP_DEV_TIMEOUT_EPILOGUE: return "device wait timed out (epilogue)";
    case B200TP_DEV_TIMEOUT_OTHER: return "device wait timed out";
    default: return "unknown status";
  }
}

const char* b200tp_last_error(void) { return last_error_cstr(); }

int b200tp_version(void) { return 100; }

size_t b200tp_flash_fwd_workspace_bytes(const b200tp_attn_args* a) {
  if (check_attn(a) != B200TP_OK) return 0;
  return pick(a) == 1 ? flash_tc_fwd_workspace_bytes(a) : 0;
}

int b200tp_flash_fwd_ws(const b200tp_attn_args* a, const void* q, const void* k, const void* v, void* o, float* lse,
                        void* workspace, size_t workspace_bytes, void* stream, int* status) {
  int rc = check_attn(a);
  if (rc) return rc;
  if (q == nullptr || k == nullptr || v == nullptr || o == nullptr || lse == nullptr)
    return fail(B200TP_ERR_ATTN_INPUT, "null tensor pointer");
  if (workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
    return fail(B200TP_ERR_WORKSPACE, "attention forward workspace must be 256-byte aligned");
  rc = require_sm100();
  if (rc) return rc;
  const int impl = pick(a);
  if (impl < 0) return B200TP_ERR_UNSUPPORTED_ATTN;
  if (impl == 1)
    return flash_tc_fwd(a, q, k, v, o, lse, workspace, workspace_bytes, static_cast<cudaStream_t>(stream), status);
  return flash_simt_fwd(a, q, k, v, o, lse, static_cast<cudaStream_t>(stream));
}

int b200tp_flash_fwd(const b200tp_attn_args* a, const void* q, const void* k, const void* v, void* o, float* lse,
                     void* stream, int* status) {
  return b200tp_flash_fwd_ws(a, q, k, v, o, lse, nullptr, 0, stream, status);
}

size_t b200tp_flash_bwd_workspace_bytes(const b200tp_attn_args* a) {
  if (check_attn(a) != B200TP_OK) return 0;
  const int impl = pick(a);
  if (impl < 0) return 0;
  if (impl == 1) return flash_tc_bwd_workspace_bytes(a);
  return align_up(static_cast<size_t>(a->b) * a->hq * a->s * sizeof(float), 256);   // CUDA-core path: the -D row vector
}

int b200tp_flash_bwd(const b200tp_attn_args* a, const void* q, const void* k, const void* v, const void* o,
                     const float* lse, const void* d_o, void* dq, void* dk, void* dv, void* workspace,
                     size_t workspace_bytes, void* stream, int* status) {
  int rc = check_attn(a);
  if (rc) return rc;
  if (q == nullptr || k == nullptr || v == nullptr || o == nullptr || lse == nullptr || d_o == nullptr ||
      dq == nullptr || dk == nullptr || dv == nullptr)
    return fail(B200TP_ERR_ATTN_INPUT, "null tensor pointer");
  rc = require_sm100();
  if (rc) return rc;
  const int impl = pick(a);
  if (impl < 0) return B200TP_ERR_UNSUPPORTED_ATTN;
  const size_t need = b200tp_flash_bwd_workspace_bytes(a);
  if (workspace == nullptr || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0 || workspace_bytes < need)
    return fail(B200TP_ERR_WORKSPACE, "attention backward workspace missing, misaligned or smaller than " +
                                          std::to_string(need) + " bytes");
  if (impl == 1)
    return flash_tc_bwd(a, q, k, v, o, lse, d_o, dq, dk, dv, workspace, static_cast<cudaStream_t>(stream), status);
  return flash_simt_bwd(a, q, k, v, o, lse, d_o, dq, dk, dv, static_cast<float*>(workspace),
                        static_cast<cudaStream_t>(stream));
}

}  // extern "C"
