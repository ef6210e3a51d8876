// CUDA-core causal / packed-segment GQA attention: forward (O, L) and backward (D, dQ,
// dK/dV).  One warp owns one output row and splits head_dim across its lanes; all
// arithmetic is fp32.  Serves fp32 tensors and head_dim 64 / 96 (the tcgen05 kernels serve
// bf16 at head_dim 128) and doubles as an independent on-device cross-check.
//
// The per-row structure follows the reference's scalar kernels
// (attention/kernel/source.py:38-174 forward, :682-797 dQ, :1221-1334 dK/dV): online
// softmax per key, GQA by kv = h / (Hq / Hkv), a key is visible iff same segment and
// j <= i, L = m + log(l) over the scaled scores.
#include "flash.h"

#include "ptx.cuh"

namespace b200tp {
namespace {

template <typename T>
__device__ __forceinline__ float ld_f32(const T* p);
template <>
__device__ __forceinline__ float ld_f32<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ld_f32<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

template <typename T>
__device__ __forceinline__ void st_f32(T* p, float v);
template <>
__device__ __forceinline__ void st_f32<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void st_f32<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct Strides {
  long long b, h, s;
};

struct SimtAttn {
  int B, Hq, Hkv, S;
  float scale;
  Strides q, k, v, o;
  const int* seg_id;
  const int* seg_start;
};

template <typename T, int EPL>
__global__ void __launch_bounds__(128)
fwd_kernel(SimtAttn a, const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, T* __restrict__ o,
           float* __restrict__ lse) {
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int h = blockIdx.y, b = blockIdx.z;
  if (i >= a.S) return;
  const int kvh = h / (a.Hq / a.Hkv);
  const T* qp = q + b * a.q.b + h * a.q.h + static_cast<long long>(i) * a.q.s + lane * EPL;
  const T* kp = k + b * a.k.b + kvh * a.k.h + lane * EPL;
  const T* vp = v + b * a.v.b + kvh * a.v.h + lane * EPL;
  float qv[EPL], acc[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    qv[e] = ld_f32(qp + e);
    acc[e] = 0.f;
  }
  int lo = 0, sid = 0;
  const int* segs = nullptr;
  if (a.seg_id != nullptr) {
    segs = a.seg_id + static_cast<long long>(b) * a.S;
    sid = segs[i];
    lo = a.seg_start[static_cast<long long>(b) * a.S + i];
    if (lo < 0) lo = 0;
    if (lo > i) lo = i;
  }
  float m = -INFINITY, l = 0.f;
  for (int j = lo; j <= i; ++j) {
    if (segs != nullptr && segs[j] != sid) continue;
    float s = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) s = fmaf(qv[e], ld_f32(kp + static_cast<long long>(j) * a.k.s + e), s);
    s = wsum(s) * a.scale;
    const float nm = fmaxf(m, s);
    const float alpha = expf(m - nm);
    const float p = expf(s - nm);
    l = l * alpha + p;
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[e] = fmaf(p, ld_f32(vp + static_cast<long long>(j) * a.v.s + e), acc[e] * alpha);
    m = nm;
  }
  T* op = o + b * a.o.b + h * a.o.h + static_cast<long long>(i) * a.o.s + lane * EPL;
  const float inv = 1.f / l;
#pragma unroll
  for (int e = 0; e < EPL; ++e) st_f32(op + e, acc[e] * inv);
  if (lane == 0) lse[(static_cast<long long>(b) * a.Hq + h) * a.S + i] = m + logf(l);
}

template <typename T, int EPL>
__global__ void __launch_bounds__(128)
bwd_d_kernel(SimtAttn a, const T* __restrict__ d_o, const T* __restrict__ o, float* __restrict__ dvec) {
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int h = blockIdx.y, b = blockIdx.z;
  if (i >= a.S) return;
  const long long off = b * a.o.b + h * a.o.h + static_cast<long long>(i) * a.o.s + lane * EPL;
  float s = 0.f;
#pragma unroll
  for (int e = 0; e < EPL; ++e) s = fmaf(ld_f32(d_o + off + e), ld_f32(o + off + e), s);
  s = wsum(s);
  if (lane == 0) dvec[(static_cast<long long>(b) * a.Hq + h) * a.S + i] = s;
}

template <typename T, int EPL>
__global__ void __launch_bounds__(128)
bwd_dq_kernel(SimtAttn a, const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
              const T* __restrict__ d_o, const float* __restrict__ lse, const float* __restrict__ dvec,
              T* __restrict__ dq) {
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int h = blockIdx.y, b = blockIdx.z;
  if (i >= a.S) return;
  const int kvh = h / (a.Hq / a.Hkv);
  const T* qp = q + b * a.q.b + h * a.q.h + static_cast<long long>(i) * a.q.s + lane * EPL;
  const T* dop = d_o + b * a.o.b + h * a.o.h + static_cast<long long>(i) * a.o.s + lane * EPL;
  const T* kp = k + b * a.k.b + kvh * a.k.h + lane * EPL;
  const T* vp = v + b * a.v.b + kvh * a.v.h + lane * EPL;
  float qv[EPL], dov[EPL], acc[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    qv[e] = ld_f32(qp + e);
    dov[e] = ld_f32(dop + e);
    acc[e] = 0.f;
  }
  const long long ri = (static_cast<long long>(b) * a.Hq + h) * a.S + i;
  const float L = lse[ri], Dv = dvec[ri];
  int lo = 0, sid = 0;
  const int* segs = nullptr;
  if (a.seg_id != nullptr) {
    segs = a.seg_id + static_cast<long long>(b) * a.S;
    sid = segs[i];
    lo = a.seg_start[static_cast<long long>(b) * a.S + i];
    if (lo < 0) lo = 0;
    if (lo > i) lo = i;
  }
  for (int j = lo; j <= i; ++j) {
    if (segs != nullptr && segs[j] != sid) continue;
    float s = 0.f, dp = 0.f;
    float kv[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      kv[e] = ld_f32(kp + static_cast<long long>(j) * a.k.s + e);
      s = fmaf(qv[e], kv[e], s);
      dp = fmaf(dov[e], ld_f32(vp + static_cast<long long>(j) * a.v.s + e), dp);
    }
    s = wsum(s) * a.scale;
    dp = wsum(dp);
    const float p = expf(s - L);
    const float ds = p * (dp - Dv);
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[e] = fmaf(ds, kv[e], acc[e]);
  }
  T* dqp = dq + b * a.q.b + h * a.q.h + static_cast<long long>(i) * a.q.s + lane * EPL;
#pragma unroll
  for (int e = 0; e < EPL; ++e) st_f32(dqp + e, acc[e] * a.scale);
}

template <typename T, int EPL>
__global__ void __launch_bounds__(128)
bwd_dkv_kernel(SimtAttn a, const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
               const T* __restrict__ d_o, const float* __restrict__ lse, const float* __restrict__ dvec,
               T* __restrict__ dk, T* __restrict__ dv) {
  const int lane = threadIdx.x & 31;
  const int j = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int kvh = blockIdx.y, b = blockIdx.z;
  if (j >= a.S) return;
  const int group = a.Hq / a.Hkv;
  const T* kp = k + b * a.k.b + kvh * a.k.h + static_cast<long long>(j) * a.k.s + lane * EPL;
  const T* vp = v + b * a.v.b + kvh * a.v.h + static_cast<long long>(j) * a.v.s + lane * EPL;
  float kv[EPL], vv[EPL], dka[EPL], dva[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    kv[e] = ld_f32(kp + e);
    vv[e] = ld_f32(vp + e);
    dka[e] = 0.f;
    dva[e] = 0.f;
  }
  const int* segs = a.seg_id != nullptr ? a.seg_id + static_cast<long long>(b) * a.S : nullptr;
  const int sid = segs != nullptr ? segs[j] : 0;
  for (int g = 0; g < group; ++g) {
    const int h = kvh * group + g;
    const T* qb = q + b * a.q.b + h * a.q.h + lane * EPL;
    const T* dob = d_o + b * a.o.b + h * a.o.h + lane * EPL;
    const long long rbase = (static_cast<long long>(b) * a.Hq + h) * a.S;
    for (int i = j; i < a.S; ++i) {
      if (segs != nullptr && segs[i] != sid) continue;
      float s = 0.f, dp = 0.f;
      float qv[EPL], dov[EPL];
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        qv[e] = ld_f32(qb + static_cast<long long>(i) * a.q.s + e);
        dov[e] = ld_f32(dob + static_cast<long long>(i) * a.o.s + e);
        s = fmaf(qv[e], kv[e], s);
        dp = fmaf(dov[e], vv[e], dp);
      }
      s = wsum(s) * a.scale;
      dp = wsum(dp);
      const float p = expf(s - lse[rbase + i]);
      const float ds = p * (dp - dvec[rbase + i]);
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        dva[e] = fmaf(p, dov[e], dva[e]);
        dka[e] = fmaf(ds, qv[e], dka[e]);
      }
    }
  }
  T* dkp = dk + b * a.k.b + kvh * a.k.h + static_cast<long long>(j) * a.k.s + lane * EPL;
  T* dvp = dv + b * a.v.b + kvh * a.v.h + static_cast<long long>(j) * a.v.s + lane * EPL;
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    st_f32(dkp + e, dka[e] * a.scale);
    st_f32(dvp + e, dva[e]);
  }
}

SimtAttn pack(const b200tp_attn_args* a) {
  SimtAttn s{};
  s.B = a->b; s.Hq = a->hq; s.Hkv = a->hkv; s.S = a->s;
  s.scale = a->scale;
  s.q = {a->q_stride[0], a->q_stride[1], a->q_stride[2]};
  s.k = {a->k_stride[0], a->k_stride[1], a->k_stride[2]};
  s.v = {a->v_stride[0], a->v_stride[1], a->v_stride[2]};
  s.o = {a->o_stride[0], a->o_stride[1], a->o_stride[2]};
  s.seg_id = a->seg_id;
  s.seg_start = a->seg_start;
  return s;
}

template <typename T, int EPL>
int fwd_t(const b200tp_attn_args* a, const void* q, const void* k, const void* v, void* o, float* lse,
          cudaStream_t stream) {
  dim3 grid((a->s + 3) / 4, a->hq, a->b);
  fwd_kernel<T, EPL><<<grid, 128, 0, stream>>>(pack(a), static_cast<const T*>(q), static_cast<const T*>(k),
                                               static_cast<const T*>(v), static_cast<T*>(o), lse);
  B200TP_CUDA_OK(cudaGetLastError());
  return B200TP_OK;
}

template <typename T, int EPL>
int bwd_t(const b200tp_attn_args* a, const void* q, const void* k, const void* v, const void* o, const float* lse,
          const void* d_o, void* dq, void* dk, void* dv, float* dvec, cudaStream_t stream) {
  const SimtAttn s = pack(a);
  dim3 gq((a->s + 3) / 4, a->hq, a->b);
  dim3 gk((a->s + 3) / 4, a->hkv, a->b);
  bwd_d_kernel<T, EPL><<<gq, 128, 0, stream>>>(s, static_cast<const T*>(d_o), static_cast<const T*>(o), dvec);
  B200TP_CUDA_OK(cudaGetLastError());
  bwd_dq_kernel<T, EPL><<<gq, 128, 0, stream>>>(s, static_cast<const T*>(q), static_cast<const T*>(k),
                                                static_cast<const T*>(v), static_cast<const T*>(d_o), lse, dvec,
                                                static_cast<T*>(dq));
  B200TP_CUDA_OK(cudaGetLastError());
  bwd_dkv_kernel<T, EPL><<<gk, 128, 0, stream>>>(s, static_cast<const T*>(q), static_cast<const T*>(k),
                                                 static_cast<const T*>(v), static_cast<const T*>(d_o), lse, dvec,
                                                 static_cast<T*>(dk), static_cast<T*>(dv));
  B200TP_CUDA_OK(cudaGetLastError());
  return B200TP_OK;
}

}  // namespace

int flash_simt_fwd(const b200tp_attn_args* a, const void* q, const void* k, const void* v, void* o, float* lse,
                   cudaStream_t stream) {
  const bool bf = a->dtype == B200TP_BF16;
  switch (a->d) {
    case 64: return bf ? fwd_t<__nv_bfloat16, 2>(a, q, k, v, o, lse, stream) : fwd_t<float, 2>(a, q, k, v, o, lse, stream);
    case 96: return bf ? fwd_t<__nv_bfloat16, 3>(a, q, k, v, o, lse, stream) : fwd_t<float, 3>(a, q, k, v, o, lse, stream);
    case 128: return bf ? fwd_t<__nv_bfloat16, 4>(a, q, k, v, o, lse, stream) : fwd_t<float, 4>(a, q, k, v, o, lse, stream);
  }
  return fail(B200TP_ERR_UNSUPPORTED_ATTN, "head_dim must be 64, 96 or 128");
}

int flash_simt_bwd(const b200tp_attn_args* a, const void* q, const void* k, const void* v, const void* o,
                   const float* lse, const void* d_o, void* dq, void* dk, void* dv, float* dvec, cudaStream_t stream) {
  const bool bf = a->dtype == B200TP_BF16;
  switch (a->d) {
    case 64:
      return bf ? bwd_t<__nv_bfloat16, 2>(a, q, k, v, o, lse, d_o, dq, dk, dv, dvec, stream)
                : bwd_t<float, 2>(a, q, k, v, o, lse, d_o, dq, dk, dv, dvec, stream);
    case 96:
      return bf ? bwd_t<__nv_bfloat16, 3>(a, q, k, v, o, lse, d_o, dq, dk, dv, dvec, stream)
                : bwd_t<float, 3>(a, q, k, v, o, lse, d_o, dq, dk, dv, dvec, stream);
    case 128:
      return bf ? bwd_t<__nv_bfloat16, 4>(a, q, k, v, o, lse, d_o, dq, dk, dv, dvec, stream)
                : bwd_t<float, 4>(a, q, k, v, o, lse, d_o, dq, dk, dv, dvec, stream);
  }
  return fail(B200TP_ERR_UNSUPPORTED_ATTN, "head_dim must be 64, 96 or 128");
}

}  // namespace b200tp
