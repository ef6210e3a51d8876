// Internal launchers of the attention kernels.
#pragma once

#include "common.h"

namespace b200tp {

// CUDA-core path: fp32 / bf16, head_dim 64 / 96 / 128.
int flash_simt_fwd(const b200tp_attn_args* a, const void* q, const void* k, const void* v, void* o, float* lse,
                   cudaStream_t stream);
int flash_simt_bwd(const b200tp_attn_args* a, const void* q, const void* k, const void* v, const void* o,
                   const float* lse, const void* d_o, void* dq, void* dk, void* dv, float* dvec, cudaStream_t stream);

// tcgen05 path: bf16, head_dim 128.
int flash_tc_fwd(const b200tp_attn_args* a, const void* q, const void* k, const void* v, void* o, float* lse,
                 cudaStream_t stream, int* status);
// dq_acc: fp32 (B, Hq, S_pad, 128) zero-initialised by the launcher; dvec: (B, Hq, S) f32.
size_t flash_tc_bwd_workspace_bytes(const b200tp_attn_args* a);
int flash_tc_bwd(const b200tp_attn_args* a, const void* q, const void* k, const void* v, const void* o,
                 const float* lse, const void* d_o, void* dq, void* dk, void* dv, void* workspace,
                 cudaStream_t stream, int* status);

}  // namespace b200tp
