// Launchers of the tcgen05 linear-cross-entropy kernels (bf16 operands, fp32 accumulate).
#pragma once

#include "common.h"

namespace b200tp {

constexpr int kCeTileRows = 128;   // rows of hidden per tile
constexpr int kCeTileCols = 256;   // vocab columns (logits) / hidden columns (dH) per tile

// A 4-bit affine group-64 head (codes (V, D/8) uint32 low nibble first, scales / biases (V, D/64) bf16
// or fp32).  Passed to the launchers below, the weight operand is expanded inside the kernels and `w`
// is ignored; a null pointer (or a null `wq`) means a dense bf16 weight matrix `w`.
struct QuantHead {
  const uint32_t* wq;
  const void* scales;
  const void* biases;
  int qp_f32;
};

// Vocab splits the forward uses for (n rows, v_rows vocab rows): one partial triple per
// (row, split) lands in the workspace.
int ce_tc_fwd_splits(int64_t n, int64_t v_rows);

// Forward partials over weight rows [vrow0, vrow1) of a (w_rows_total, d) bf16 matrix whose
// row 0 has global vocab id `vocab_id0`.  pm/ps/pt: [splits][n] f32.
int ce_tc_launch_fwd(const void* hidden, const void* w, int64_t w_rows_total, int64_t n, int d, int64_t vrow0,
                     int64_t vrow1, int64_t vocab_id0, const int64_t* targets, int64_t ignore_index, int splits,
                     float* pm, float* ps, float* pt, const QuantHead* q, cudaStream_t stream, int* status);

// g[n][ldg] (bf16) = (exp(z - lse) - onehot) * ct over weight rows [vrow0, vrow1); columns
// up to the next multiple of 256 are written (zeros past vrow1).
int ce_tc_launch_bwd_g(const void* hidden, const void* w, int64_t w_rows_total, int64_t n, int d, int64_t vrow0,
                       int64_t vrow1, int64_t vocab_id0, const int64_t* targets, int64_t ignore_index,
                       const float* lse, const float* ct, void* g, int ldg, const QuantHead* q, cudaStream_t stream,
                       int* status);

// dH = [acc_in +] G[:, :k_total] @ W[wrow0 : wrow0 + k_total, :]; written to acc_out (f32)
// and/or out_bf16.  k_total is a multiple of 64; rows of W past w_rows_total read as zero.
// The 128 x 256 output tiles are numbered row-block-major; this launch computes tiles
// [tile0, tile1) (negative: from the first / through the last).  `ce_tc_dh_rows_done(n, d, t)` is
// the number of leading rows of d_hidden that are complete once tiles [0, t) have run.
int ce_tc_dh_tiles(int64_t n, int d);
int ce_tc_dh_rows_done(int64_t n, int d, int tiles_done);
int ce_tc_launch_dh(const void* g, int ldg, int k_total, int64_t n, const void* w, int64_t w_rows_total, int d,
                    int64_t wrow0, const float* acc_in, float* acc_out, void* out_bf16, int tile0, int tile1,
                    const QuantHead* q, cudaStream_t stream, int* status);

// d_weight block (v_rows, d) bf16 = G[:, :v_rows]^T @ hidden: g (n, ldg) bf16 as written by
// ce_tc_launch_bwd_g, hidden (n, d) bf16.  fp32 accumulation over the n rows, one rounding.
int ce_tc_launch_dw(const void* g, int ldg, int64_t v_rows, int64_t n, const void* hidden, int d, void* d_weight_block,
                    cudaStream_t stream, int* status);

}  // namespace b200tp
