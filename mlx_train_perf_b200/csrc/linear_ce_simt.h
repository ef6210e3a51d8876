// CUDA-core linear-cross-entropy chunk steps and the kernels shared with the tcgen05 path.
#pragma once

#include "common.h"

namespace b200tp {

// Merge `parts` (max, sum-exp, target) triples per row; part p of each array lies `stride`
// floats after part 0.  Any output pointer may be null.  targets may be null (no masking).
int launch_combine(const float* pm, const float* ps, const float* pt, int64_t stride, int parts, int64_t n,
                   const int64_t* targets, int64_t ignore_index, float* row_max, float* row_sumexp, float* tgt_out,
                   float* lse_out, float* nll_out, cudaStream_t stream);

// out3 = {masked sum of nll, masked mean, number of rows whose target != ignore_index}; fixed summation order.
int launch_loss_reduce(const float* nll, const int64_t* targets, int64_t n, int64_t ignore_index, float* out3,
                       cudaStream_t stream);
// ct[i] = upstream[0] (/ max(count[0], 1) when count != null) on non-ignored rows, 0 elsewhere.
int launch_loss_cotangent(const int64_t* targets, int64_t n, int64_t ignore_index, const float* upstream,
                          const float* count, float* ct, cudaStream_t stream);

int launch_dequant_int4(const uint32_t* w_q, const void* scales, const void* biases, int qparam_dtype, int64_t row0,
                        int64_t rows, int d, int group, void* out, int out_dtype, cudaStream_t stream);

// logits_ws (n, width) f32 = hidden @ w_chunk^T, folded into run_m / run_s / run_t.
int ce_simt_fwd_chunk(const void* hidden, const void* w_chunk, int dtype, int64_t n, int d, int64_t width,
                      int64_t vocab_id0, const int64_t* targets, int64_t ignore_index, float* logits_ws, float* run_m,
                      float* run_s, float* run_t, int first, cudaStream_t stream);

// dh_acc (n, d) f32 (+)= g @ w_chunk with g formed in logits_ws.
int ce_simt_bwd_chunk(const void* hidden, const void* w_chunk, int dtype, int64_t n, int d, int64_t width,
                      int64_t vocab_id0, const int64_t* targets, int64_t ignore_index, const float* lse,
                      const float* ct, float* logits_ws, float* dh_acc, int accumulate, cudaStream_t stream);

// d_weight block (width, d) in the hidden dtype = g^T @ hidden, g (n, width) f32 as left in
// logits_ws by ce_simt_bwd_chunk.
int ce_simt_dw_chunk(const float* g_ws, int64_t width, const void* hidden, int dtype, int64_t n, int d,
                     void* d_weight_block, cudaStream_t stream);

int launch_cast_f32_to_bf16(const float* src, void* dst, int64_t count, cudaStream_t stream);

}  // namespace b200tp
