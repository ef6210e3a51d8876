// CUDA-core (SIMT) linear cross-entropy path and the small kernels both paths share.
//
// The SIMT path serves fp32 heads (exact fp32 FMA accumulation, which the tensor cores do
// not offer) and shapes the tcgen05 path refuses (D not a multiple of 8).  It streams the
// vocabulary in chunks through an (N, chunk) fp32 scratch tile -- the structure of the
// reference's pure-array implementation, core/chunked.py:35-90 -- and so never holds (N, V).
//
// Shared kernels: `combine_kernel` merges per-split (max, sum-exp, target) triples into
// lse / nll (the logaddexp merge of core/chunked.py:43), `dequant_int4_kernel` expands the
// 4-bit affine group layout of core/kernel/source.py:193-208.
#include "linear_ce_simt.h"

#include "ptx.cuh"

namespace b200tp {

namespace {

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

constexpr int TS = 64;  // tile side
constexpr int TK = 16;

// C[m][n] = sum_k A[m][k] * B[n][k]      (A: M x K, B: Nn x K, both row-major)
template <typename TA, typename TB>
__global__ void __launch_bounds__(256)
gemm_nt_kernel(const TA* __restrict__ A, long long lda, const TB* __restrict__ B, long long ldb, float* __restrict__ C,
               long long ldc, int M, int Nn, int K) {
  __shared__ float As[TK][TS + 1];
  __shared__ float Bs[TK][TS + 1];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * TS, n0 = blockIdx.x * TS;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += TK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = threadIdx.x + i * 256;
      const int r = idx >> 4, c = idx & 15;
      As[c][r] = (m0 + r < M && k0 + c < K) ? to_f32(A[static_cast<long long>(m0 + r) * lda + k0 + c]) : 0.f;
      Bs[c][r] = (n0 + r < Nn && k0 + c < K) ? to_f32(B[static_cast<long long>(n0 + r) * ldb + k0 + c]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < Nn) C[static_cast<long long>(m) * ldc + n] = acc[i][j];
    }
  }
}

// C[m][n] (+)= sum_k A[m][k] * B[k][n]   (A: M x K fp32, B: K x Nn row-major)
template <typename TB>
__global__ void __launch_bounds__(256)
gemm_nn_acc_kernel(const float* __restrict__ A, long long lda, const TB* __restrict__ B, long long ldb,
                   float* __restrict__ C, long long ldc, int M, int Nn, int K, int accumulate) {
  __shared__ float As[TK][TS + 1];
  __shared__ float Bs[TK][TS + 1];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * TS, n0 = blockIdx.x * TS;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += TK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = threadIdx.x + i * 256;
      const int r = idx >> 4, c = idx & 15;  // A: r = row, c = k
      As[c][r] = (m0 + r < M && k0 + c < K) ? A[static_cast<long long>(m0 + r) * lda + k0 + c] : 0.f;
      const int kr = idx >> 6, nc = idx & 63;  // B: kr = k, nc = column
      Bs[kr][nc] = (k0 + kr < K && n0 + nc < Nn) ? to_f32(B[static_cast<long long>(k0 + kr) * ldb + n0 + nc]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < Nn) {
        float* dst = C + static_cast<long long>(m) * ldc + n;
        *dst = accumulate ? (*dst + acc[i][j]) : acc[i][j];
      }
    }
  }
}

// C[M x Nn] = A^T B with A (K x M) fp32 row-major (the g scratch), B (K x Nn) row-major
// (hidden); written once in the output type.  d_weight of a trainable head, one vocab chunk.
template <typename TB, typename TO>
__global__ void __launch_bounds__(256)
gemm_tn_out_kernel(const float* __restrict__ A, long long lda, const TB* __restrict__ B, long long ldb,
                   TO* __restrict__ C, long long ldc, int M, int Nn, int K) {
  __shared__ float As[TK][TS + 1];
  __shared__ float Bs[TK][TS + 1];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * TS, n0 = blockIdx.x * TS;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += TK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = threadIdx.x + i * 256;
      const int kr = idx >> 6, c = idx & 63;  // kr = k, c = column of A (m) / of B (n)
      As[kr][c] = (k0 + kr < K && m0 + c < M) ? A[static_cast<long long>(k0 + kr) * lda + m0 + c] : 0.f;
      Bs[kr][c] = (k0 + kr < K && n0 + c < Nn) ? to_f32(B[static_cast<long long>(k0 + kr) * ldb + n0 + c]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < Nn) C[static_cast<long long>(m) * ldc + n] = static_cast<TO>(acc[i][j]);
    }
  }
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One warp per row: fold a chunk of logits into the running (max, sum-exp, target logit).
__global__ void __launch_bounds__(256)
rows_fwd_kernel(const float* __restrict__ logits, long long ld, int n_rows, int width, long long vocab_id0,
                const long long* __restrict__ targets, long long ignore_index, float* run_m, float* run_s,
                float* run_t, int first) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= n_rows) return;
  const float* z = logits + static_cast<long long>(row) * ld;
  float m = -INFINITY;
  for (int c = lane; c < width; c += 32) m = fmaxf(m, z[c]);
  m = warp_max(m);
  float s = 0.f;
  for (int c = lane; c < width; c += 32) s += expf(z[c] - m);
  s = warp_sum(s);
  if (lane == 0) {
    float om = first ? -INFINITY : run_m[row];
    float os = first ? 0.f : run_s[row];
    float ot = first ? 0.f : run_t[row];
    const float nm = fmaxf(om, m);
    os = os * expf(om - nm) + s * expf(m - nm);
    const long long t = targets[row];
    if (t != ignore_index) {
      const long long rel = t - vocab_id0;
      if (rel >= 0 && rel < width) ot = z[rel];
    }
    run_m[row] = nm;
    run_s[row] = os;
    run_t[row] = ot;
  }
}

// In place: z -> g = (exp(z - lse) - onehot) * ct, optionally rounded through bf16.
template <bool ROUND_BF16>
__global__ void __launch_bounds__(256)
rows_bwd_kernel(float* __restrict__ logits, long long ld, int n_rows, int width, long long vocab_id0,
                const long long* __restrict__ targets, long long ignore_index, const float* __restrict__ lse,
                const float* __restrict__ ct) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= n_rows) return;
  float* z = logits + static_cast<long long>(row) * ld;
  const long long t = targets[row];
  const bool valid = t != ignore_index;
  const float c_row = valid ? ct[row] : 0.f;
  const float l = lse[row];
  const long long rel = valid ? t - vocab_id0 : -1;
  for (int c = lane; c < width; c += 32) {
    float g = expf(z[c] - l);
    if (c == rel) g -= 1.f;
    g *= c_row;
    if (ROUND_BF16) g = __bfloat162float(__float2bfloat16_rn(g));
    z[c] = g;
  }
}

__global__ void cast_out_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long count) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < count) dst[i] = __float2bfloat16_rn(src[i]);
}

// Merge `parts` triples per row.  pm/ps/pt point at part 0; part p is `stride` floats on.
__global__ void combine_kernel(const float* __restrict__ pm, const float* __restrict__ ps, const float* __restrict__ pt,
                               long long stride, int parts, long long n, const long long* __restrict__ targets,
                               long long ignore_index, float* row_max, float* row_sumexp, float* tgt_out, float* lse_out,
                               float* nll_out) {
  const long long row = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (row >= n) return;
  float m = -INFINITY;
  for (int p = 0; p < parts; ++p) m = fmaxf(m, pm[p * stride + row]);
  float s = 0.f, t = 0.f;
  for (int p = 0; p < parts; ++p) {
    const float pmv = pm[p * stride + row];
    const float psv = ps[p * stride + row];
    if (psv > 0.f) s += psv * expf(pmv - m);
    t += pt[p * stride + row];
  }
  const bool valid = targets == nullptr || targets[row] != ignore_index;
  if (!valid) t = 0.f;
  const float lse = m + logf(s);
  if (row_max != nullptr) row_max[row] = m;
  if (row_sumexp != nullptr) row_sumexp[row] = s;
  if (tgt_out != nullptr) tgt_out[row] = t;
  if (lse_out != nullptr) lse_out[row] = lse;
  if (nll_out != nullptr) nll_out[row] = valid ? lse - t : 0.f;
}

// Masked reduction of the per-row losses (the masked mean of adapters/mlx_lm.py:192-216 of the
// reference): out = {sum of nll over rows whose target != ignore_index, that sum / max(count, 1),
// count}.  One block; every thread sums its rows in index order and the block adds the thread sums in a
// fixed tree, so the result does not depend on scheduling.
constexpr int kReduceThreads = 1024;
__global__ void __launch_bounds__(kReduceThreads)
loss_reduce_kernel(const float* __restrict__ nll, const long long* __restrict__ targets, long long n,
                   long long ignore_index, float* __restrict__ out3) {
  __shared__ float s_sum[kReduceThreads];
  __shared__ float s_cnt[kReduceThreads];
  float sum = 0.f, cnt = 0.f;
  for (long long i = threadIdx.x; i < n; i += kReduceThreads) {
    const bool valid = targets == nullptr || targets[i] != ignore_index;
    if (valid) {
      sum += nll[i];
      cnt += 1.f;
    }
  }
  s_sum[threadIdx.x] = sum;
  s_cnt[threadIdx.x] = cnt;
  __syncthreads();
  for (int ofs = kReduceThreads / 2; ofs > 0; ofs >>= 1) {
    if (threadIdx.x < ofs) {
      s_sum[threadIdx.x] += s_sum[threadIdx.x + ofs];
      s_cnt[threadIdx.x] += s_cnt[threadIdx.x + ofs];
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    out3[0] = s_sum[0];
    out3[1] = s_sum[0] / fmaxf(s_cnt[0], 1.f);
    out3[2] = s_cnt[0];
  }
}

// Cotangent of the per-row losses under a reduced loss: ct[i] = upstream * (divide ? 1 / max(count, 1) : 1)
// on rows whose target != ignore_index, 0 elsewhere; `upstream` and `count` are device scalars.
__global__ void __launch_bounds__(256)
loss_cotangent_kernel(const long long* __restrict__ targets, long long n, long long ignore_index,
                      const float* __restrict__ upstream, const float* __restrict__ count, float* __restrict__ ct) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float g = upstream[0];
  if (count != nullptr) g = g / fmaxf(count[0], 1.f);
  ct[i] = (targets == nullptr || targets[i] != ignore_index) ? g : 0.f;
}

// One thread per packed word (8 codes).
template <typename TP, typename TO>
__global__ void dequant_int4_kernel(const uint32_t* __restrict__ wq, const TP* __restrict__ scales,
                                    const TP* __restrict__ biases, long long row0, long long rows, int d, int group,
                                    TO* __restrict__ out) {
  const int words = d / 8;
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= rows * words) return;
  const long long r = i / words;
  const int wi = static_cast<int>(i - r * words);
  const long long src_row = row0 + r;
  const uint32_t word = wq[src_row * words + wi];
  const int g = (wi * 8) / group;
  const float sc = to_f32(scales[src_row * (d / group) + g]);
  const float bi = to_f32(biases[src_row * (d / group) + g]);
  TO* dst = out + r * d + wi * 8;
  float w[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) w[k] = fmaf(sc, static_cast<float>((word >> (4 * k)) & 0xFu), bi);
  // one (bf16) or two (fp32) 16-byte stores per thread: `out` is 256-byte aligned and d % 8 == 0
  if constexpr (sizeof(TO) == 2) {
    *reinterpret_cast<uint4*>(dst) = make_uint4(pack_bf16x2(w[0], w[1]), pack_bf16x2(w[2], w[3]),
                                                pack_bf16x2(w[4], w[5]), pack_bf16x2(w[6], w[7]));
  } else {
    *reinterpret_cast<float4*>(dst) = make_float4(w[0], w[1], w[2], w[3]);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(w[4], w[5], w[6], w[7]);
  }
}

// One 32-byte store (a whole sector); `p` 32-byte aligned.
__device__ __forceinline__ void st_global_32b(void* p, const uint32_t (&v)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]),
               "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}

// Four packed words (32 codes of one group) per thread: one 16-byte load, one scale / bias pair, and the
// thread's 64 (bf16) or 128 (fp32) contiguous output bytes as whole 32-byte sectors (`st.global.v8.b32`).
// Needs d % 32 == 0, group % 32 == 0 and 32-byte aligned output rows.  (A variant whose warps wrote 512
// contiguous bytes per store instruction from four words 32 apart needed four scale / bias pairs per thread
// and was a third slower.)
template <typename TP, typename TO>
__global__ void __launch_bounds__(256)
dequant_int4_x4_kernel(const uint32_t* __restrict__ wq, const TP* __restrict__ scales, const TP* __restrict__ biases,
                       long long row0, long long rows, int d, int group, TO* __restrict__ out) {
  const int quads = d / 32;
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= rows * quads) return;
  const long long r = i / quads;
  const int qi = static_cast<int>(i - r * quads);
  const long long src_row = row0 + r;
  const uint4 words = *reinterpret_cast<const uint4*>(wq + src_row * (d / 8) + qi * 4);
  const int g = (qi * 32) / group;
  const float sc = to_f32(scales[src_row * (d / group) + g]);
  const float bi = to_f32(biases[src_row * (d / group) + g]);
  const uint32_t wv[4] = {words.x, words.y, words.z, words.w};
  TO* dst = out + r * d + qi * 32;
  if constexpr (sizeof(TO) == 2) {
#pragma unroll
    for (int j = 0; j < 4; j += 2) {
      uint32_t o[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint32_t word = wv[j + (k >> 2)];
        const int sh = 8 * (k & 3);
        o[k] = pack_bf16x2(fmaf(sc, static_cast<float>((word >> sh) & 0xFu), bi),
                           fmaf(sc, static_cast<float>((word >> (sh + 4)) & 0xFu), bi));
      }
      st_global_32b(dst + j * 8, o);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t o[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) o[k] = __float_as_uint(fmaf(sc, static_cast<float>((wv[j] >> (4 * k)) & 0xFu), bi));
      st_global_32b(dst + j * 8, o);
    }
  }
}

template <typename TP, typename TO>
void launch_dequant_typed(const uint32_t* w_q, const void* scales, const void* biases, int64_t row0, int64_t rows, int d,
                          int group, void* out, cudaStream_t stream) {
  const bool wide = d % 32 == 0 && group % 32 == 0 && (reinterpret_cast<uintptr_t>(w_q) & 15) == 0 &&
                    (reinterpret_cast<uintptr_t>(out) & 31) == 0;
  const int threads = 256;
  if (wide) {
    const unsigned blocks = static_cast<unsigned>(ceil_div(rows * (d / 32), threads));
    dequant_int4_x4_kernel<TP, TO><<<blocks, threads, 0, stream>>>(w_q, static_cast<const TP*>(scales),
                                                                   static_cast<const TP*>(biases), row0, rows, d, group,
                                                                   static_cast<TO*>(out));
  } else {
    const unsigned blocks = static_cast<unsigned>(ceil_div(rows * (d / 8), threads));
    dequant_int4_kernel<TP, TO><<<blocks, threads, 0, stream>>>(w_q, static_cast<const TP*>(scales),
                                                                static_cast<const TP*>(biases), row0, rows, d, group,
                                                                static_cast<TO*>(out));
  }
}

}  // namespace

int launch_combine(const float* pm, const float* ps, const float* pt, int64_t stride, int parts, int64_t n,
                   const int64_t* targets, int64_t ignore_index, float* row_max, float* row_sumexp, float* tgt_out,
                   float* lse_out, float* nll_out, cudaStream_t stream) {
  if (n <= 0) return B200TP_OK;
  const int threads = 256;
  const unsigned blocks = static_cast<unsigned>(ceil_div(n, threads));
  combine_kernel<<<blocks, threads, 0, stream>>>(pm, ps, pt, stride, parts, n,
                                                 reinterpret_cast<const long long*>(targets), ignore_index, row_max,
                                                 row_sumexp, tgt_out, lse_out, nll_out);
  B200TP_CUDA_OK(cudaGetLastError());
  return B200TP_OK;
}

int launch_loss_reduce(const float* nll, const int64_t* targets, int64_t n, int64_t ignore_index, float* out3,
                       cudaStream_t stream) {
  loss_reduce_kernel<<<1, kReduceThreads, 0, stream>>>(nll, reinterpret_cast<const long long*>(targets), n,
                                                       ignore_index, out3);
  B200TP_CUDA_OK(cudaGetLastError());
  return B200TP_OK;
}

int launch_loss_cotangent(const int64_t* targets, int64_t n, int64_t ignore_index, const float* upstream,
                          const float* count, float* ct, cudaStream_t stream) {
  loss_cotangent_kernel<<<static_cast<unsigned>(ceil_div(n, 256)), 256, 0, stream>>>(
      reinterpret_cast<const long long*>(targets), n, ignore_index, upstream, count, ct);
  B200TP_CUDA_OK(cudaGetLastError());
  return B200TP_OK;
}

int launch_dequant_int4(const uint32_t* w_q, const void* scales, const void* biases, int qparam_dtype, int64_t row0,
                        int64_t rows, int d, int group, void* out, int out_dtype, cudaStream_t stream) {
  if (rows <= 0) return B200TP_OK;
  if (qparam_dtype == B200TP_BF16 && out_dtype == B200TP_BF16)
    launch_dequant_typed<__nv_bfloat16, __nv_bfloat16>(w_q, scales, biases, row0, rows, d, group, out, stream);
  else if (qparam_dtype == B200TP_BF16 && out_dtype == B200TP_F32)
    launch_dequant_typed<__nv_bfloat16, float>(w_q, scales, biases, row0, rows, d, group, out, stream);
  else if (qparam_dtype == B200TP_F32 && out_dtype == B200TP_BF16)
    launch_dequant_typed<float, __nv_bfloat16>(w_q, scales, biases, row0, rows, d, group, out, stream);
  else
    launch_dequant_typed<float, float>(w_q, scales, biases, row0, rows, d, group, out, stream);
  B200TP_CUDA_OK(cudaGetLastError());
  return B200TP_OK;
}

int ce_simt_fwd_chunk(const void* hidden, const void* w_chunk, int dtype, int64_t n, int d, int64_t width,
                      int64_t vocab_id0, const int64_t* targets, int64_t ignore_index, float* logits_ws, float* run_m,
                      float* run_s, float* run_t, int first, cudaStream_t stream) {
  dim3 grid(static_cast<unsigned>(ceil_div(width, TS)), static_cast<unsigned>(ceil_div(n, TS)));
  if (dtype == B200TP_F32)
    gemm_nt_kernel<float, float><<<grid, 256, 0, stream>>>(static_cast<const float*>(hidden), d,
                                                           static_cast<const float*>(w_chunk), d, logits_ws, width,
                                                           static_cast<int>(n), static_cast<int>(width), d);
  else
    gemm_nt_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(hidden), d, static_cast<const __nv_bfloat16*>(w_chunk), d, logits_ws, width,
        static_cast<int>(n), static_cast<int>(width), d);
  B200TP_CUDA_OK(cudaGetLastError());
  rows_fwd_kernel<<<static_cast<unsigned>(ceil_div(n, 8)), 256, 0, stream>>>(
      logits_ws, width, static_cast<int>(n), static_cast<int>(width), vocab_id0,
      reinterpret_cast<const long long*>(targets), ignore_index, run_m, run_s, run_t, first);
  B200TP_CUDA_OK(cudaGetLastError());
  return B200TP_OK;
}

int ce_simt_bwd_chunk(const void* hidden, const void* w_chunk, int dtype, int64_t n, int d, int64_t width,
                      int64_t vocab_id0, const int64_t* targets, int64_t ignore_index, const float* lse,
                      const float* ct, float* logits_ws, float* dh_acc, int accumulate, cudaStream_t stream) {
  dim3 grid(static_cast<unsigned>(ceil_div(width, TS)), static_cast<unsigned>(ceil_div(n, TS)));
  dim3 grid2(static_cast<unsigned>(ceil_div(d, TS)), static_cast<unsigned>(ceil_div(n, TS)));
  const unsigned row_blocks = static_cast<unsigned>(ceil_div(n, 8));
  if (dtype == B200TP_F32) {
    gemm_nt_kernel<float, float><<<grid, 256, 0, stream>>>(static_cast<const float*>(hidden), d,
                                                           static_cast<const float*>(w_chunk), d, logits_ws, width,
                                                           static_cast<int>(n), static_cast<int>(width), d);
    B200TP_CUDA_OK(cudaGetLastError());
    rows_bwd_kernel<false><<<row_blocks, 256, 0, stream>>>(logits_ws, width, static_cast<int>(n),
                                                           static_cast<int>(width), vocab_id0,
                                                           reinterpret_cast<const long long*>(targets), ignore_index,
                                                           lse, ct);
    B200TP_CUDA_OK(cudaGetLastError());
    gemm_nn_acc_kernel<float><<<grid2, 256, 0, stream>>>(logits_ws, width, static_cast<const float*>(w_chunk), d,
                                                         dh_acc, d, static_cast<int>(n), d, static_cast<int>(width),
                                                         accumulate);
  } else {
    gemm_nt_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(hidden), d, static_cast<const __nv_bfloat16*>(w_chunk), d, logits_ws, width,
        static_cast<int>(n), static_cast<int>(width), d);
    B200TP_CUDA_OK(cudaGetLastError());
    rows_bwd_kernel<true><<<row_blocks, 256, 0, stream>>>(logits_ws, width, static_cast<int>(n),
                                                          static_cast<int>(width), vocab_id0,
                                                          reinterpret_cast<const long long*>(targets), ignore_index,
                                                          lse, ct);
    B200TP_CUDA_OK(cudaGetLastError());
    gemm_nn_acc_kernel<__nv_bfloat16><<<grid2, 256, 0, stream>>>(
        logits_ws, width, static_cast<const __nv_bfloat16*>(w_chunk), d, dh_acc, d, static_cast<int>(n), d,
        static_cast<int>(width), accumulate);
  }
  B200TP_CUDA_OK(cudaGetLastError());
  return B200TP_OK;
}

int ce_simt_dw_chunk(const float* g_ws, int64_t width, const void* hidden, int dtype, int64_t n, int d,
                     void* d_weight_block, cudaStream_t stream) {
  dim3 grid(static_cast<unsigned>(ceil_div(d, TS)), static_cast<unsigned>(ceil_div(width, TS)));
  if (dtype == B200TP_F32) {
    gemm_tn_out_kernel<float, float><<<grid, 256, 0, stream>>>(g_ws, width, static_cast<const float*>(hidden), d,
                                                               static_cast<float*>(d_weight_block), d,
                                                               static_cast<int>(width), d, static_cast<int>(n));
  } else {
    gemm_tn_out_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, stream>>>(
        g_ws, width, static_cast<const __nv_bfloat16*>(hidden), d, static_cast<__nv_bfloat16*>(d_weight_block), d,
        static_cast<int>(width), d, static_cast<int>(n));
  }
  B200TP_CUDA_OK(cudaGetLastError());
  return B200TP_OK;
}

int launch_cast_f32_to_bf16(const float* src, void* dst, int64_t count, cudaStream_t stream) {
  if (count <= 0) return B200TP_OK;
  cast_out_kernel<<<static_cast<unsigned>(ceil_div(count, 256)), 256, 0, stream>>>(
      src, static_cast<__nv_bfloat16*>(dst), count);
  B200TP_CUDA_OK(cudaGetLastError());
  return B200TP_OK;
}

}  // namespace b200tp
