// In-kernel expansion of a 4-bit affine group-64 head: one (vocab row, group of 64 input columns)
// -> 64 bf16 weights written straight into the 128-byte-swizzled shared-memory row a tcgen05
// operand descriptor expects.  Layout of the packed head: core/kernel/source.py:193-208 of the
// reference (8 codes per uint32, low nibble first; w = scale * code + bias per group).
//
// Rounding contract, shared with dequant_int4_kernel and the CPU oracle: w = fma(scale, code, bias)
// evaluated in fp32, rounded ONCE to bf16.  For bf16 scales / biases the fast path below gets the
// same bits with two packed bf16 instructions per code pair: (128 + code) is built exactly from the
// nibble with a byte permute and one logic op (0x4300 | code is the bf16 of 128 + code), 128 is
// subtracted exactly, and fma.rn.bf16x2 rounds the exact scale * code + bias once.  That equals the
// double rounding through fp32 whenever the fp32 fma is itself exact or the code term cannot reach a
// rounding boundary, which holds unless the bias is non-zero and more than eight binades below the
// scale (spread of the exact sum <= 24 bits otherwise; see `dq_fast_ok`); such degenerate groups,
// and fp32 scales / biases, take the fp32 path.
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

namespace b200tp {

struct QRow {
  uint4 lo, hi;        // the group's eight code words
  uint32_t sc, bi;     // raw scale / bias: a bf16 in the low half, or fp32 bits (qparams fp32)
};

__device__ __forceinline__ float fma_rn_exact(float a, float b, float c) {
  float d;
  asm("fma.rn.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));   // no flush-to-zero, whatever the flags
  return d;
}

__device__ __forceinline__ bool dq_fast_ok(uint32_t sc_bits, uint32_t bi_bits) {
  const uint32_t es = (sc_bits >> 7) & 0xFFu, eb = (bi_bits >> 7) & 0xFFu;
  return (bi_bits & 0x7FFFu) == 0u || eb + 8u >= es;
}

// Eight codes of one word -> four bf16 pairs (one 16-byte chunk).
__device__ __forceinline__ uint4 dq_word_fast(uint32_t w, __nv_bfloat162 s2, __nv_bfloat162 b2) {
  const uint32_t ws = w >> 4;
  const __nv_bfloat162 k128 = __floats2bfloat162_rn(128.f, 128.f);
  uint32_t out[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    // bytes: [w.byte j, w.byte j, ws.byte j, ws.byte j]; the low nibbles are codes 2j and 2j + 1
    const uint32_t t = __byte_perm(w, ws, j | (j << 4) | ((4 + j) << 8) | ((4 + j) << 12));
    const uint32_t x = (t & 0x000F000Fu) | 0x43004300u;
    __nv_bfloat162 c2 = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&x), k128);
    __nv_bfloat162 o = __hfma2(s2, c2, b2);
    out[j] = *reinterpret_cast<uint32_t*>(&o);
  }
  return make_uint4(out[0], out[1], out[2], out[3]);
}

__device__ __forceinline__ uint4 dq_word_f32(uint32_t w, float sc, float bi) {
  uint32_t out[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float a = fma_rn_exact(sc, static_cast<float>((w >> (8 * j)) & 0xFu), bi);
    const float b = fma_rn_exact(sc, static_cast<float>((w >> (8 * j + 4)) & 0xFu), bi);
    __nv_bfloat162 o = __floats2bfloat162_rn(a, b);
    out[j] = *reinterpret_cast<uint32_t*>(&o);
  }
  return make_uint4(out[0], out[1], out[2], out[3]);
}

// `row_smem`: start of the 128-byte row (inside a 1024-byte aligned swizzle atom); `r7` = row & 7.
// `valid` false writes zeros (rows past the end of the head).
__device__ __forceinline__ void dq_store_row(uint8_t* row_smem, int r7, const QRow& q, bool qp_f32, bool valid) {
  const uint32_t w[8] = {q.lo.x, q.lo.y, q.lo.z, q.lo.w, q.hi.x, q.hi.y, q.hi.z, q.hi.w};
  if (!valid) {
#pragma unroll
    for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(row_smem + ((c ^ r7) << 4)) = make_uint4(0u, 0u, 0u, 0u);
    return;
  }
  if (!qp_f32 && dq_fast_ok(q.sc, q.bi)) {
    const uint32_t s2b = (q.sc & 0xFFFFu) | (q.sc << 16), b2b = (q.bi & 0xFFFFu) | (q.bi << 16);
    const __nv_bfloat162 s2 = *reinterpret_cast<const __nv_bfloat162*>(&s2b);
    const __nv_bfloat162 b2 = *reinterpret_cast<const __nv_bfloat162*>(&b2b);
#pragma unroll
    for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(row_smem + ((c ^ r7) << 4)) = dq_word_fast(w[c], s2, b2);
  } else {
    const float sc = qp_f32 ? __uint_as_float(q.sc) : __uint_as_float(q.sc << 16);
    const float bi = qp_f32 ? __uint_as_float(q.bi) : __uint_as_float(q.bi << 16);
#pragma unroll
    for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(row_smem + ((c ^ r7) << 4)) = dq_word_f32(w[c], sc, bi);
  }
}

// Loads of one (row, group): `words` = w_q + row * (D / 8) + group * 8 (32-byte aligned).
__device__ __forceinline__ void dq_load_row(QRow& q, const uint32_t* words, const void* scales, const void* biases,
                                            long long qidx, bool qp_f32) {
  const uint4* p = reinterpret_cast<const uint4*>(words);
  q.lo = __ldg(p);
  q.hi = __ldg(p + 1);
  if (qp_f32) {
    q.sc = __ldg(reinterpret_cast<const uint32_t*>(scales) + qidx);
    q.bi = __ldg(reinterpret_cast<const uint32_t*>(biases) + qidx);
  } else {
    q.sc = __ldg(reinterpret_cast<const unsigned short*>(scales) + qidx);
    q.bi = __ldg(reinterpret_cast<const unsigned short*>(biases) + qidx);
  }
}

}  // namespace b200tp
