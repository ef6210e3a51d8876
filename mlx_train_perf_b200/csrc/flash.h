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
// The forward splits every query block's key range over several CTAs when the grid would otherwise
// leave SMs idle (see fwd_splits in flash_tc.cu); that needs `flash_tc_fwd_workspace_bytes` of scratch
// (0 when it would not split).  Without a workspace that large it runs unsplit.
size_t flash_tc_fwd_workspace_bytes(const b200tp_attn_args* a);
int flash_tc_fwd(const b200tp_attn_args* a, const void* q, const void* k, const void* v, void* o, float* lse,
                 void* workspace, size_t workspace_bytes, cudaStream_t stream, int* status);
size_t flash_tc_bwd_workspace_bytes(const b200tp_attn_args* a);
int flash_tc_bwd(const b200tp_attn_args* a, const void* q, const void* k, const void* v, const void* o,
                 const float* lse, const void* d_o, void* dq, void* dk, void* dv, void* workspace,
                 cudaStream_t stream, int* status);

}  // namespace b200tp
