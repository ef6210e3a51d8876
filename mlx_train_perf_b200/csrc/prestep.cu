// Attention pre-step: per-head RMSNorm (optional) followed by rotary position embedding, forward
// and backward, on (B, L, H, d) views with arbitrary (B, L, H) strides -- the step the reference's
// wrapper runs between the q / k projections and the attention operator
// (attention/wrapper.py:133-157: `mx.fast.rms_norm` per head, then `rope`).
//
// One warp per token, looping over its heads; d in {64, 96, 128}.  The rotation pairs element j with
// j + d/2 (the "rotate half" convention: y = n cos + [-n_hi, n_lo] sin), so a lane owns whole
// pairs.  All arithmetic is fp32 with one rounding to the output type.  HBM-bound: every vector
// is read once and written once; cos / sin / weight are read once per token.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../../include/b200tp.h"
#include "common.h"

namespace b200tp {
namespace {

// Eight adjacent elements per access (16 bytes for bf16, 2 x 16 for fp32).
__device__ __forceinline__ void ld8(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void st8(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void st8(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}

// sum over the 8-lane group of this lane
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct PreParams {
  int B, L, H, d;
  long long x_sb, x_sl, x_sh;
  long long y_sb, y_sl, y_sh;
  long long cs_sb, cs_sl;
  float eps;
};

// One warp per TOKEN.  The warp's four 8-lane groups work on four heads at a time; lane q of a
// group owns elements [8q, 8q + 8) of the low half of the head vector and their rotation partners
// in the high half (groups use 4 / 6 / 8 lanes for d = 64 / 96 / 128).  cos / sin of the position
// and the norm weight are read once per token; every head vector is read once and written once
// with 16-byte accesses.
// T: tensor type, TC: cos / sin type.  NORM: apply RMSNorm with `weight` first.
template <typename T, typename TC, bool NORM>
__global__ void __launch_bounds__(256)
norm_rope_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, const T* __restrict__ weight,
                     const TC* __restrict__ cosp, const TC* __restrict__ sinp, const PreParams p) {
  const int lane = threadIdx.x & 31;
  const long long tok = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (tok >= static_cast<long long>(p.B) * p.L) return;
  const int l = static_cast<int>(tok % p.L);
  const int b = static_cast<int>(tok / p.L);
  const int half = p.d / 2;
  const int g = lane >> 3, j = (lane & 7) * 8;
  const bool act = j < half;
  float c_lo[8], c_hi[8], s_lo[8], s_hi[8], w_lo[8], w_hi[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) c_lo[e] = c_hi[e] = s_lo[e] = s_hi[e] = 0.f, w_lo[e] = w_hi[e] = 1.f;
  if (act) {
    const TC* cv = cosp + b * p.cs_sb + l * p.cs_sl;
    const TC* sv = sinp + b * p.cs_sb + l * p.cs_sl;
    ld8(cv + j, c_lo);
    ld8(cv + j + half, c_hi);
    ld8(sv + j, s_lo);
    ld8(sv + j + half, s_hi);
    if (NORM) {
      ld8(weight + j, w_lo);
      ld8(weight + j + half, w_hi);
    }
  }
  const T* xt = x + b * p.x_sb + l * p.x_sl;
  T* yt = y + b * p.y_sb + l * p.y_sl;
  const float inv_d = 1.f / static_cast<float>(p.d);
  for (int h0 = 0; h0 < p.H; h0 += 4) {
    const int h = h0 + g;
    const bool on = act && h < p.H;
    float lo[8], hi[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) lo[e] = hi[e] = 0.f;
    if (on) {
      ld8(xt + h * p.x_sh + j, lo);
      ld8(xt + h * p.x_sh + j + half, hi);
    }
    float r = 1.f;
    if (NORM) {
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += lo[e] * lo[e] + hi[e] * hi[e];
      r = rsqrtf(group_sum(ss) * inv_d + p.eps);
    }
    if (on) {
      float o_lo[8], o_hi[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float n1 = NORM ? lo[e] * r * w_lo[e] : lo[e];
        const float n2 = NORM ? hi[e] * r * w_hi[e] : hi[e];
        o_lo[e] = n1 * c_lo[e] - n2 * s_lo[e];
        o_hi[e] = n2 * c_hi[e] + n1 * s_hi[e];
      }
      st8(yt + h * p.y_sh + j, o_lo);
      st8(yt + h * p.y_sh + j + half, o_hi);
    }
  }
}

// Backward: dx from dy; d_weight partial sums (one row of d floats per block) when NORM.
// Persistent blocks: warp w of block b handles tokens b * 8 + w, then strides by gridDim * 8.
template <typename T, typename TC, bool NORM, bool WANT_DW>
__global__ void __launch_bounds__(256)
norm_rope_bwd_kernel(const T* __restrict__ x, const T* __restrict__ dy, T* __restrict__ dx,
                     const T* __restrict__ weight, const TC* __restrict__ cosp, const TC* __restrict__ sinp,
                     float* __restrict__ dw_part, const PreParams p) {
  __shared__ float dw_sm[WANT_DW ? 8 : 1][4][128];   // [warp][head slot][element]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int half = p.d / 2;
  const int g = lane >> 3, j = (lane & 7) * 8;
  const bool act = j < half;
  const float inv_d = 1.f / static_cast<float>(p.d);
  float w_lo[8], w_hi[8], dw_lo[8], dw_hi[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) w_lo[e] = w_hi[e] = 1.f, dw_lo[e] = dw_hi[e] = 0.f;
  if (NORM && act) {
    ld8(weight + j, w_lo);
    ld8(weight + j + half, w_hi);
  }
  const long long tokens = static_cast<long long>(p.B) * p.L;
  for (long long tok = static_cast<long long>(blockIdx.x) * 8 + warp; tok < tokens;
       tok += static_cast<long long>(gridDim.x) * 8) {
    const int l = static_cast<int>(tok % p.L);
    const int b = static_cast<int>(tok / p.L);
    float c_lo[8], c_hi[8], s_lo[8], s_hi[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) c_lo[e] = c_hi[e] = s_lo[e] = s_hi[e] = 0.f;
    if (act) {
      const TC* cv = cosp + b * p.cs_sb + l * p.cs_sl;
      const TC* sv = sinp + b * p.cs_sb + l * p.cs_sl;
      ld8(cv + j, c_lo);
      ld8(cv + j + half, c_hi);
      ld8(sv + j, s_lo);
      ld8(sv + j + half, s_hi);
    }
    const T* xt = x + b * p.x_sb + l * p.x_sl;
    T* dxt = dx + b * p.x_sb + l * p.x_sl;
    const T* dyt = dy + b * p.y_sb + l * p.y_sl;
    for (int h0 = 0; h0 < p.H; h0 += 4) {
      const int h = h0 + g;
      const bool on = act && h < p.H;
      float xl[8], xh[8], gl[8], gh[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) xl[e] = xh[e] = gl[e] = gh[e] = 0.f;
      if (on) {
        float d1[8], d2[8];
        ld8(dyt + h * p.y_sh + j, d1);
        ld8(dyt + h * p.y_sh + j + half, d2);
        if (NORM) {
          ld8(xt + h * p.x_sh + j, xl);
          ld8(xt + h * p.x_sh + j + half, xh);
        }
        // transpose of the rotation: dn_lo = dy_lo cos_lo + dy_hi sin_hi; dn_hi = dy_hi cos_hi - dy_lo sin_lo
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          gl[e] = d1[e] * c_lo[e] + d2[e] * s_hi[e];
          gh[e] = d2[e] * c_hi[e] - d1[e] * s_lo[e];
        }
      }
      if (!NORM) {
        if (on) {
          st8(dxt + h * p.x_sh + j, gl);
          st8(dxt + h * p.x_sh + j + half, gh);
        }
        continue;
      }
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += xl[e] * xl[e] + xh[e] * xh[e];
      const float r = rsqrtf(group_sum(ss) * inv_d + p.eps);
      float dot = 0.f;   // sum over d of (dn * w) * xhat
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float h1 = xl[e] * r, h2 = xh[e] * r;      // xhat
        if (WANT_DW) {
          dw_lo[e] += gl[e] * h1;
          dw_hi[e] += gh[e] * h2;
        }
        dot += gl[e] * w_lo[e] * h1 + gh[e] * w_hi[e] * h2;
      }
      const float m = group_sum(dot) * inv_d;
      if (on) {
        float o_lo[8], o_hi[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          o_lo[e] = r * (gl[e] * w_lo[e] - xl[e] * r * m);
          o_hi[e] = r * (gh[e] * w_hi[e] - xh[e] * r * m);
        }
        st8(dxt + h * p.x_sh + j, o_lo);
        st8(dxt + h * p.x_sh + j + half, o_hi);
      }
    }
  }
  if (NORM && WANT_DW) {
    // block partial of d_weight: sum the 8 warps x 4 head slots in a fixed order
    if (act) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        dw_sm[warp][g][j + e] = dw_lo[e];
        dw_sm[warp][g][j + half + e] = dw_hi[e];
      }
    }
    __syncthreads();
    for (int q = threadIdx.x; q < p.d; q += blockDim.x) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w)
#pragma unroll
        for (int k = 0; k < 4; ++k) s += dw_sm[w][k][q];
      dw_part[static_cast<long long>(blockIdx.x) * p.d + q] = s;
    }
  }
}

// Sum of the per-block weight-gradient partials, [blocks][d] -> [d].  One block per 32 columns, 32 x 32
// threads: thread (tx, ty) adds rows ty, ty + 32, ... of its column (coalesced over tx), the 32 row sums
// of a column then meet in shared memory and are added in index order -- a fixed order, so the result is
// bitwise reproducible.  (A single block of d threads walking all rows serially took as long as the
// backward kernel itself.)
__global__ void __launch_bounds__(1024)
dw_reduce_kernel(const float* __restrict__ part, int blocks, int d, float* __restrict__ out) {
  __shared__ float sm[32][33];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int j = blockIdx.x * 32 + tx;
  float s = 0.f;
  if (j < d)
    for (int b = ty; b < blocks; b += 32) s += part[static_cast<long long>(b) * d + j];
  sm[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && j < d) {
    float t = 0.f;
#pragma unroll
    for (int r = 0; r < 32; ++r) t += sm[r][tx];
    out[j] = t;
  }
}

int check(const b200tp_prestep_args* a) {
  if (a == nullptr) return fail(B200TP_ERR_ATTN_INPUT, "args is null");
  if (a->b < 1 || a->l < 1 || a->h < 1) return fail(B200TP_ERR_ATTN_INPUT, "b, l, h must be positive");
  if (a->d != 64 && a->d != 96 && a->d != 128)
    return fail(B200TP_ERR_UNSUPPORTED_ATTN, "head_dim must be 64, 96 or 128");
  if (a->dtype != B200TP_F32 && a->dtype != B200TP_BF16) return fail(B200TP_ERR_ATTN_INPUT, "dtype must be f32 or bf16");
  if (a->cs_dtype != B200TP_F32 && a->cs_dtype != B200TP_BF16)
    return fail(B200TP_ERR_ATTN_INPUT, "cos / sin dtype must be f32 or bf16");
  if (a->cos == nullptr || a->sin == nullptr) return fail(B200TP_ERR_ATTN_INPUT, "cos / sin is null");
  // elements are accessed eight at a time with 16-byte loads and stores
  for (int i = 0; i < 3; ++i)
    if (a->x_stride[i] % 8 != 0 || a->y_stride[i] % 8 != 0)
      return fail(B200TP_ERR_ATTN_INPUT, "tensor strides must be multiples of 8 elements");
  if (a->cs_stride_b % 8 != 0 || a->cs_stride_l % 8 != 0)
    return fail(B200TP_ERR_ATTN_INPUT, "cos / sin strides must be multiples of 8 elements");
  if ((reinterpret_cast<uintptr_t>(a->cos) & 15) != 0 || (reinterpret_cast<uintptr_t>(a->sin) & 15) != 0 ||
      (reinterpret_cast<uintptr_t>(a->weight) & 15) != 0)
    return fail(B200TP_ERR_ATTN_INPUT, "cos / sin / weight must be 16-byte aligned");
  return B200TP_OK;
}

PreParams params(const b200tp_prestep_args* a) {
  PreParams p{};
  p.B = a->b; p.L = a->l; p.H = a->h; p.d = a->d;
  p.x_sb = a->x_stride[0]; p.x_sl = a->x_stride[1]; p.x_sh = a->x_stride[2];
  p.y_sb = a->y_stride[0]; p.y_sl = a->y_stride[1]; p.y_sh = a->y_stride[2];
  p.cs_sb = a->cs_stride_b; p.cs_sl = a->cs_stride_l;
  p.eps = a->eps;
  return p;
}

int bwd_blocks(const b200tp_prestep_args* a) {
  const long long tokens = static_cast<long long>(a->b) * a->l;
  const long long want = (tokens + 7) / 8;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  return static_cast<int>(want < cap ? want : cap);
}

template <typename T, typename TC>
int launch_fwd(const b200tp_prestep_args* a, const void* x, void* y, cudaStream_t stream) {
  const PreParams p = params(a);
  const long long tokens = static_cast<long long>(a->b) * a->l;
  const unsigned blocks = static_cast<unsigned>((tokens + 7) / 8);
  if (a->weight != nullptr)
    norm_rope_fwd_kernel<T, TC, true><<<blocks, 256, 0, stream>>>(
        static_cast<const T*>(x), static_cast<T*>(y), static_cast<const T*>(a->weight),
        static_cast<const TC*>(a->cos), static_cast<const TC*>(a->sin), p);
  else
    norm_rope_fwd_kernel<T, TC, false><<<blocks, 256, 0, stream>>>(
        static_cast<const T*>(x), static_cast<T*>(y), nullptr, static_cast<const TC*>(a->cos),
        static_cast<const TC*>(a->sin), p);
  B200TP_CUDA_OK(cudaGetLastError());
  return B200TP_OK;
}

template <typename T, typename TC>
int launch_bwd(const b200tp_prestep_args* a, const void* x, const void* dy, void* dx, float* d_weight, float* ws,
               cudaStream_t stream) {
  const PreParams p = params(a);
  const int blocks = bwd_blocks(a);
  const T* xp = static_cast<const T*>(x);
  const T* dyp = static_cast<const T*>(dy);
  T* dxp = static_cast<T*>(dx);
  const TC* cp = static_cast<const TC*>(a->cos);
  const TC* sp = static_cast<const TC*>(a->sin);
  if (a->weight != nullptr && d_weight != nullptr) {
    norm_rope_bwd_kernel<T, TC, true, true><<<blocks, 256, 0, stream>>>(xp, dyp, dxp, static_cast<const T*>(a->weight),
                                                                        cp, sp, ws, p);
    B200TP_CUDA_OK(cudaGetLastError());
    dw_reduce_kernel<<<(a->d + 31) / 32, dim3(32, 32), 0, stream>>>(ws, blocks, a->d, d_weight);
  } else if (a->weight != nullptr) {
    norm_rope_bwd_kernel<T, TC, true, false><<<blocks, 256, 0, stream>>>(xp, dyp, dxp, static_cast<const T*>(a->weight),
                                                                         cp, sp, nullptr, p);
  } else {
    norm_rope_bwd_kernel<T, TC, false, false><<<blocks, 256, 0, stream>>>(xp, dyp, dxp, nullptr, cp, sp, nullptr, p);
  }
  B200TP_CUDA_OK(cudaGetLastError());
  return B200TP_OK;
}

}  // namespace
}  // namespace b200tp

extern "C" {

int b200tp_qk_norm_rope_fwd(const b200tp_prestep_args* a, const void* x, void* y, void* stream_v) {
  using namespace b200tp;
  int rc = check(a);
  if (rc) return rc;
  if (x == nullptr || y == nullptr) return fail(B200TP_ERR_ATTN_INPUT, "x / y is null");
  if (((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) != 0)
    return fail(B200TP_ERR_ATTN_INPUT, "x / y must be 16-byte aligned");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (a->dtype == B200TP_BF16)
    return a->cs_dtype == B200TP_BF16 ? launch_fwd<__nv_bfloat16, __nv_bfloat16>(a, x, y, stream)
                                      : launch_fwd<__nv_bfloat16, float>(a, x, y, stream);
  return a->cs_dtype == B200TP_BF16 ? launch_fwd<float, __nv_bfloat16>(a, x, y, stream)
                                    : launch_fwd<float, float>(a, x, y, stream);
}

size_t b200tp_qk_norm_rope_bwd_workspace_bytes(const b200tp_prestep_args* a) {
  using namespace b200tp;
  if (check(a) != B200TP_OK) return 0;
  if (a->weight == nullptr) return 0;
  return align_up(static_cast<size_t>(bwd_blocks(a)) * a->d * sizeof(float), 256);
}

int b200tp_qk_norm_rope_bwd(const b200tp_prestep_args* a, const void* x, const void* dy, void* dx, float* d_weight,
                            void* workspace, size_t workspace_bytes, void* stream_v) {
  using namespace b200tp;
  int rc = check(a);
  if (rc) return rc;
  if (x == nullptr || dy == nullptr || dx == nullptr) return fail(B200TP_ERR_ATTN_INPUT, "x / dy / dx is null");
  if (((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dx)) & 15) != 0)
    return fail(B200TP_ERR_ATTN_INPUT, "x / dy / dx must be 16-byte aligned");
  if (d_weight != nullptr && a->weight == nullptr)
    return fail(B200TP_ERR_ATTN_INPUT, "d_weight requested without a norm weight");
  if (d_weight != nullptr) {
    const size_t need = b200tp_qk_norm_rope_bwd_workspace_bytes(a);
    if (workspace == nullptr || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0 || workspace_bytes < need)
      return fail(B200TP_ERR_WORKSPACE, "pre-step backward workspace missing, misaligned or too small");
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  float* ws = static_cast<float*>(workspace);
  if (a->dtype == B200TP_BF16)
    return a->cs_dtype == B200TP_BF16 ? launch_bwd<__nv_bfloat16, __nv_bfloat16>(a, x, dy, dx, d_weight, ws, stream)
                                      : launch_bwd<__nv_bfloat16, float>(a, x, dy, dx, d_weight, ws, stream);
  return a->cs_dtype == B200TP_BF16 ? launch_bwd<float, __nv_bfloat16>(a, x, dy, dx, d_weight, ws, stream)
                                    : launch_bwd<float, float>(a, x, dy, dx, d_weight, ws, stream);
}

}  // extern "C"
