/*
 * b200tp -- C ABI of the B200 (sm_100a) fused linear-cross-entropy and flash-attention
 * kernels.  One shared library, plain pointers and sizes, no framework types.
 *
 * Conventions
 *   - Every pointer is a caller-owned DEVICE pointer valid on `stream` unless stated.
 *   - Calls enqueue work on `stream` and return without synchronising.  The library never
 *     allocates device memory: scratch comes in through `workspace` (size from the matching
 *     *_workspace_bytes function; 256-byte aligned).
 *   - Return value: 0 on success, a B200TP_ERR_* code on a refusal (nothing was launched).
 *   - `status` is a device int the kernels write when a bounded device-side wait gave up
 *     (see B200TP_DEV_*); callers zero it once and read it whenever they synchronise.
 *   - dtype codes: B200TP_F32 = 0, B200TP_BF16 = 1.
 *
 * The reference these entry points stand in for is a pure-Python package without an FFI of
 * its own; each function cites the Python launcher it replaces
 * (paths under src/mlx_train_perf/).
 */
#ifndef B200TP_H_
#define B200TP_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200TP_F32 0
#define B200TP_BF16 1

/* host-side refusals (nothing launched) */
#define B200TP_OK 0
#define B200TP_ERR_LOSS_INPUT 1        /* maps to LossInputError */
#define B200TP_ERR_UNSUPPORTED_HEAD 2  /* maps to UnsupportedHeadError */
#define B200TP_ERR_ATTN_INPUT 3        /* maps to AttentionInputError */
#define B200TP_ERR_UNSUPPORTED_ATTN 4  /* maps to UnsupportedAttentionError */
#define B200TP_ERR_WORKSPACE 5         /* workspace missing, misaligned or too small */
#define B200TP_ERR_CUDA 6              /* a CUDA runtime / driver call failed */
#define B200TP_ERR_NO_DEVICE 7         /* current device is not compute capability 10.x */

/* device-side status words (written into `status`) */
#define B200TP_DEV_TIMEOUT_PRODUCER 101
#define B200TP_DEV_TIMEOUT_MMA 102
#define B200TP_DEV_TIMEOUT_EPILOGUE 103
#define B200TP_DEV_TIMEOUT_OTHER 104

/* implementation selectors */
#define B200TP_IMPL_AUTO 0   /* tcgen05 path for bf16 (head_dim 128 for attention), SIMT otherwise */
#define B200TP_IMPL_TC 1     /* tcgen05 / TMEM / TMA kernels; refuses what they cannot serve */
#define B200TP_IMPL_SIMT 2   /* CUDA-core fp32-accumulate kernels (fp32 inputs, odd shapes) */

const char* b200tp_status_string(int code);
const char* b200tp_last_error(void); /* thread-local detail text of the last refusal */
int b200tp_version(void);

/* ---------------------------------------------------------------------------------------
 * Fused linear cross-entropy
 * ------------------------------------------------------------------------------------- */

typedef struct b200tp_ce_args {
  /* hidden (N, D) row-major, `dtype` (f32 or bf16) */
  const void* hidden;
  /* dense head: weight (V_local, D) row-major, same dtype as hidden; NULL for a quantized head */
  const void* weight;
  /* 4-bit affine head (quant_bits == 4): codes (V_local, D/8) uint32, low nibble first;
   * scales / biases (V_local, D/group) bf16 (or f32 when qparam_dtype == B200TP_F32) */
  const uint32_t* w_q;
  const void* scales;
  const void* biases;
  /* targets (N,) int64; a row whose target == ignore_index is masked (NLL 0, no gradient) */
  const int64_t* targets;
  int64_t n;          /* rows */
  int32_t d;          /* hidden size */
  int64_t v_local;    /* vocab rows held by this call */
  int64_t v_offset;   /* global vocab id of local row 0 (vocab-sharded callers), else 0 */
  int32_t dtype;      /* B200TP_F32 | B200TP_BF16 */
  int32_t quant_bits; /* 0 (dense) | 4 */
  int32_t group_size; /* 64 when quant_bits == 4 */
  int32_t qparam_dtype;
  int64_t ignore_index;
  int32_t impl;       /* B200TP_IMPL_* */
  int32_t reserved;   /* low 16 bits: 0, or an upper bound on the vocab rows per tensor-core backward chunk in units
                       * of 256 (default: 16384 rows, fewer when N is so large that an (N, chunk) bf16 matrix would exceed
                       * 512 MiB): the backward's scratch is that matrix, so
                       * a smaller bound trades launches for memory.  4-bit heads on the tensor-core path:
                       * 0x10000 expands the head inside the kernels whatever N is, 0x20000 always dequantises chunk
                       * by chunk into the workspace (default: the forward expands inside the kernel for N <= 512,
                       * where that is the cheaper form and needs no weight scratch, and is chunked beyond; the
                       * backward is chunked at every N) */
} b200tp_ce_args;

/* Forward: per-row log-sum-exp pieces and target logit over this call's vocab rows.  A 4-bit head is
 * expanded either inside the tensor-core kernels, tile by tile in shared memory (it then never exists as a
 * bf16 matrix in global memory and needs no scratch beyond the partial triples; w_q 16-byte aligned), or
 * chunk by chunk into the workspace ahead of the dense kernels; both give the same bits
 * (w = fma(scale, code, bias) in fp32, rounded once to bf16).  See `reserved` for the choice.
 *   row_max, row_sumexp : (N,) f32, max logit and sum exp(logit - max)   [always written]
 *   tgt_logit           : (N,) f32, logit of the target if it lies in this shard, else 0
 *   lse, nll            : (N,) f32, may be NULL (vocab-sharded callers combine first);
 *                         lse = max + log(sumexp); nll = lse - tgt (0 on ignored rows)
 * Replaces core/kernel/launch.py:75-100 (`forward`, 19 chained vocab-tile dispatches) and
 * core/kernel/launch.py:336-373 (`forward_quantized`); outputs follow the residual
 * contract of core/loss.py:235-250 (nll, lse, tgt). */
size_t b200tp_linear_ce_fwd_workspace_bytes(const b200tp_ce_args* a);
int b200tp_linear_ce_fwd(const b200tp_ce_args* a, float* row_max, float* row_sumexp, float* tgt_logit,
                         float* lse, float* nll, void* workspace, size_t workspace_bytes, void* stream,
                         int* status);

/* Forward for callers that cannot allocate device memory (no cudaMalloc available to them: the
 * GPU's memory belongs to a framework pool they have no handle to, or an allocation's implicit
 * device synchronisation is unaffordable where they run).  Same outputs as
 * b200tp_linear_ce_fwd, but the per-split partial triples live in a fixed
 * B200TP_STATIC_SCRATCH_BYTES array inside the library instead of a caller workspace; the call
 * performs no allocation of any kind.  Dense bf16 heads on the tensor-core path only; a shape
 * whose partials (3 x splits x N floats) exceed the array is refused with
 * B200TP_ERR_WORKSPACE.  All calls on a device share the array (nothing in it needs clearing:
 * every slot read is written earlier in the same call), so calls that overlap on the GPU race
 * and must be ordered by the caller.  The first call on each device looks the array's address
 * up (cudaGetSymbolAddress) and should be made before any stream capture begins.
 * This entry point has no counterpart in the reference. */
#define B200TP_STATIC_SCRATCH_BYTES (6u << 20)
int b200tp_linear_ce_fwd_static(const b200tp_ce_args* a, float* row_max, float* row_sumexp, float* tgt_logit,
                                float* lse, float* nll, void* stream, int* status);

/* Merge R vocab-shard triples laid out as parts[r][3][N] (max, sumexp, tgt) into lse / nll /
 * tgt.  New (the reference is single-device); the arithmetic is the logaddexp merge of
 * core/chunked.py:43 and core/kernel/source.py:148-165. */
int b200tp_linear_ce_combine(const float* parts, int32_t num_parts, int64_t n, const int64_t* targets,
                             int64_t ignore_index, float* lse, float* nll, float* tgt_logit, void* stream);

/* Reduced loss of a trainer: out3 (device, 3 floats) = {sum of nll over the rows whose target != ignore_index,
 * that sum / max(count, 1), count}; `targets` may be NULL (no row masked).  One launch, summation in a fixed
 * order (bitwise reproducible).  Replaces the masked mean the reference's loss shim applies outside the
 * operator, adapters/mlx_lm.py:192-216 (`(ce * mask).sum() / ntoks`). */
int b200tp_linear_ce_reduce(const float* nll, const int64_t* targets, int64_t n, int64_t ignore_index, float* out3,
                            void* stream);

/* Its backward: cotangent (N,) f32 of the per-row losses = upstream[0] (/ max(count[0], 1) when `count` is not
 * NULL: the mean) on the rows whose target != ignore_index, 0 elsewhere; `upstream` and `count` are device
 * scalars (count = out3 + 2 of the reduce call).  The vector feeds b200tp_linear_ce_bwd. */
int b200tp_linear_ce_cotangent(const int64_t* targets, int64_t n, int64_t ignore_index, const float* upstream,
                               const float* count, float* cotangent, void* stream);

/* Backward to d_hidden from the SAVED global lse:
 *   g = (exp(z - lse) - onehot(target)) * cotangent;  d_hidden (+)= g @ W_local
 * cotangent (N,) f32 is the upstream gradient of the per-row NLL (rows with
 * target == ignore_index are treated as 0 regardless).  g is rounded to the weight dtype
 * before the second GEMM, accumulation is fp32 and d_hidden is cast once at the end --
 * core/chunked.py:52-90 (`chunked_backward`), the backward the reference ships, and
 * core/kernel/launch.py:181-234 (`backward_dhidden_mma`).
 *   d_hidden_dtype: hidden dtype, or B200TP_F32 for an fp32 partial (vocab-sharded callers
 *   sum partials across ranks before casting).  accumulate != 0 adds into an f32 d_hidden. */
size_t b200tp_linear_ce_bwd_workspace_bytes(const b200tp_ce_args* a, int32_t d_hidden_dtype);
int b200tp_linear_ce_bwd(const b200tp_ce_args* a, const float* lse, const float* cotangent, void* d_hidden,
                         int32_t d_hidden_dtype, int32_t accumulate, void* workspace, size_t workspace_bytes,
                         void* stream, int* status);

/* The same backward issued in `num_stages` calls, for vocab-sharded callers that overlap the cross-rank
 * reduction of the fp32 partial d_hidden with its computation (new: the reference is single-device).
 * Stage 0 launches everything up to and including the first slab of the last vocab chunk's
 * d_hidden GEMM, stage s > 0 its slab s; the slabs are whole waves of that GEMM's row-block-major
 * tile order, so splitting costs no extra tile.  `*rows_done` (host) receives the number of leading
 * rows of d_hidden that are final once the stage's launches have run: the caller may reduce rows
 * [previous rows_done, rows_done) on another stream while it issues the next stage.  All stages take
 * the same arguments and workspace; num_stages = 1 is b200tp_linear_ce_bwd.  On the CUDA-core path
 * stage 0 does all the work. */
int b200tp_linear_ce_bwd_stage(const b200tp_ce_args* a, const float* lse, const float* cotangent, void* d_hidden,
                               int32_t d_hidden_dtype, int32_t accumulate, int32_t num_stages, int32_t stage,
                               int64_t* rows_done, void* workspace, size_t workspace_bytes, void* stream,
                               int* status);

/* Backward of a TRAINABLE dense head: d_hidden exactly as b200tp_linear_ce_bwd, plus
 *   d_weight (V_local, D), weight dtype, row-major = g^T @ hidden
 * with the same g (rounded to the weight dtype), fp32 accumulation over the N rows and one
 * rounding -- the `d_w_chunks` of core/chunked.py:84-90; replaces core/kernel/launch.py:249-322
 * (`backward_dw`).  Every vocab row belongs to one chunk, so d_weight is written, never
 * accumulated; vocab-sharded callers own disjoint row blocks.  Same workspace as the plain
 * backward.  Quantized heads are frozen and are refused. */
int b200tp_linear_ce_bwd_train(const b200tp_ce_args* a, const float* lse, const float* cotangent, void* d_hidden,
                               int32_t d_hidden_dtype, int32_t accumulate, void* d_weight, void* workspace,
                               size_t workspace_bytes, void* stream, int* status);

/* Dequantise rows [row0, row0 + rows) of a 4-bit affine head into `out` (rows, D) bf16/f32:
 * w = scale * code + bias in fp32, rounded once; `out` 16-byte aligned.  core/kernel/source.py:193-208. */
int b200tp_dequant_int4(const uint32_t* w_q, const void* scales, const void* biases, int32_t qparam_dtype,
                        int64_t row0, int64_t rows, int32_t d, int32_t group_size, void* out,
                        int32_t out_dtype, void* stream);

/* Self-test of the bounded device-side wait (no counterpart in the reference, whose Metal kernels
 * have no inter-role waits).  Launches one CTA that waits on a barrier nothing completes: after
 * the library's wait limit (2 s) the kernel records B200TP_DEV_TIMEOUT_OTHER in `status` and
 * returns normally.  `waited_ns` (device, 2 x uint64, may be NULL) receives how long the waiting
 * role and a second role, released by the first one's abort, waited.  The context stays usable. */
int b200tp_selftest_bounded_wait(unsigned long long* waited_ns, void* stream, int* status);

/* ---------------------------------------------------------------------------------------
 * Flash attention (causal, GQA, optional packed segments)
 * ------------------------------------------------------------------------------------- */

typedef struct b200tp_attn_args {
  /* q/o/dq/do: (B, Hq, S, d) ; k/v/dk/dv: (B, Hkv, S, d); element strides below, the
   * innermost (d) stride must be 1.  `dtype` f32 or bf16. */
  int32_t b, hq, hkv, s, d;
  int32_t dtype;
  int64_t q_stride[3];  /* strides of (B, H, S) in elements */
  int64_t k_stride[3];
  int64_t v_stride[3];
  int64_t o_stride[3];
  float scale;
  int32_t causal;       /* must be 1 */
  /* packed segments: int32 (B, S) contiguous, or NULL.  Key j is visible to query i iff
   * seg_id[j] == seg_id[i] and j <= i; seg_start[i] = first index of i's segment. */
  const int32_t* seg_id;
  const int32_t* seg_start;
  int32_t impl;
  int32_t reserved;     /* 0; tensor-core forward only: low two bits 1 / 2 force its single-tile / two-tile
                         * kernel, bits 3-5 a split over keys into that many (2-4) shares (needs the forward workspace);
                         * tensor-core backward: 64 / 128 force dK / dV CTAs per q head / per GQA group; 256 / 512
                         * leave out the dK, dV kernel / the dQ kernel (their outputs stay unwritten: timing only) */
} b200tp_attn_args;

/* Forward: O (dtype, o_stride) and L (B, Hq, S) f32 contiguous = natural-log LSE of the
 * scaled masked scores.  Replaces attention/kernel/launch.py:386-441 (`launch_flash_fwd`). */
int b200tp_flash_fwd(const b200tp_attn_args* a, const void* q, const void* k, const void* v, void* o,
                     float* lse, void* stream, int* status);

/* The same forward with scratch.  A grid of few heads and one long sequence (one kv-head group per
 * GPU, say) leaves SMs idle and is bound by the serial chain of its longest query block; given
 * `b200tp_flash_fwd_workspace_bytes` of 256-byte-aligned workspace (0 when the shape does not need
 * it) the tensor-core path splits every query block's key range over 2-4 CTAs (fp32 partial O plus
 * a running max and sum per row) and a combine pass writes O and L.  With a NULL or smaller workspace
 * it behaves as b200tp_flash_fwd.  Bits 3-5 of `reserved` force 2-4 shares (cross-checks). */
size_t b200tp_flash_fwd_workspace_bytes(const b200tp_attn_args* a);
int b200tp_flash_fwd_ws(const b200tp_attn_args* a, const void* q, const void* k, const void* v, void* o,
                        float* lse, void* workspace, size_t workspace_bytes, void* stream, int* status);

/* Backward from saved O and L.  dq has q's strides, dk/dv have k's / v's strides, d_o has
 * o's strides.  Replaces attention/kernel/launch.py:765-787 (`launch_bwd_D`), :985-1049
 * (`launch_bwd_dq`) and :1225-1293 (`launch_bwd_dkv`).  Workspace holds the row statistics
 * of the backward (the (B,Hq,S) f32 vector D on the CUDA-core path; on the tensor-core path D and L / scale
 * as a bf16 operand tile of 32 bytes per query row, which the dQ kernel writes and the dK / dV kernel
 * multiplies into its products) and, for GQA on the tensor-core path when every q head has its own
 * dK / dV CTAs, the fp32 per-q-head dK / dV partials that are summed over the group at the end. */
size_t b200tp_flash_bwd_workspace_bytes(const b200tp_attn_args* a);
int b200tp_flash_bwd(const b200tp_attn_args* a, const void* q, const void* k, const void* v, const void* o,
                     const float* lse, const void* d_o, void* dq, void* dk, void* dv, void* workspace,
                     size_t workspace_bytes, void* stream, int* status);

/* ---------------------------------------------------------------------------------------
 * Attention pre-step: per-head RMSNorm (optional) + rotary position embedding
 * ------------------------------------------------------------------------------------- */

typedef struct b200tp_prestep_args {
  /* x, y, dy, dx: (B, L, H, d) views, `dtype` f32 or bf16, unit d stride; x / dx use x_stride,
   * y / dy use y_stride (element strides of B, L, H).  y may alias x. */
  int32_t b, l, h, d;   /* d in {64, 96, 128} */
  int32_t dtype;
  int64_t x_stride[3];
  int64_t y_stride[3];
  /* RMSNorm over d with this (d,) weight of the tensor dtype and `eps`; NULL: no norm */
  const void* weight;
  float eps;
  /* cos / sin: (L, d) rows (cs_stride_b == 0) or (B, L, d), `cs_dtype` f32 or bf16, unit d
   * stride; element j rotates with element j + d/2 ("rotate half"):
   *   y[j] = n[j] cos[j] - n[j + d/2] sin[j];  y[j + d/2] = n[j + d/2] cos[j + d/2] + n[j] sin[j + d/2] */
  const void* cos;
  const void* sin;
  int32_t cs_dtype;
  int64_t cs_stride_b, cs_stride_l;
} b200tp_prestep_args;

/* y = rope(rms_norm(x) * weight): fp32 arithmetic, one rounding.  Replaces the per-head
 * `mx.fast.rms_norm` + `rope` pair of attention/wrapper.py:133-157 (q and k are two calls). */
int b200tp_qk_norm_rope_fwd(const b200tp_prestep_args* a, const void* x, void* y, void* stream);

/* dx from dy (and d_weight (d,) f32, written, when non-NULL: needs the workspace; the partial
 * sums are reduced in a fixed order).  The reference gets this from MLX autodiff. */
size_t b200tp_qk_norm_rope_bwd_workspace_bytes(const b200tp_prestep_args* a);
int b200tp_qk_norm_rope_bwd(const b200tp_prestep_args* a, const void* x, const void* dy, void* dx, float* d_weight,
                            void* workspace, size_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* B200TP_H_ */
