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
//
// The packed codes reach the expanding threads through shared memory: the TMA producer copies them
// tile by tile (tensor maps over the uint32 words, swizzled), so no per-thread global load of codes
// exists -- 256 threads each reading their own 32 bytes of a different row cost more L1 tag look-ups
// per pipeline stage than the stage lasts.
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

namespace b200tp {

// Explicit shared-state-space accesses (32-bit shared addresses): the tile these stores fill is read by
// the tensor core through the async proxy, and the proxy fence that publishes them is qualified
// `.shared::cta`, so the stores must be shared-space instructions, not generic ones that merely happen
// to resolve to shared memory.
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr)
               : "memory");
  return v;
}

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

// `row_smem`: shared-space address of the 128-byte row (inside a 1024-byte aligned swizzle atom); `r7` = row & 7.
// `lo` / `hi`: the group's eight code words; `sc` / `bi`: raw scale / bias (a bf16 in the low half, or
// fp32 bits when `qp_f32`).  `valid` false writes zeros (rows past the end of the head).
__device__ __forceinline__ void dq_store_row(uint32_t row_smem, int r7, uint4 lo, uint4 hi, uint32_t sc_bits,
                                             uint32_t bi_bits, bool qp_f32, bool valid) {
  const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
  if (!valid) {
#pragma unroll
    for (int c = 0; c < 8; ++c) sts128(row_smem + ((c ^ r7) << 4), make_uint4(0u, 0u, 0u, 0u));
    return;
  }
  if (!qp_f32 && dq_fast_ok(sc_bits, bi_bits)) {
    const uint32_t s2b = (sc_bits & 0xFFFFu) | (sc_bits << 16), b2b = (bi_bits & 0xFFFFu) | (bi_bits << 16);
    const __nv_bfloat162 s2 = *reinterpret_cast<const __nv_bfloat162*>(&s2b);
    const __nv_bfloat162 b2 = *reinterpret_cast<const __nv_bfloat162*>(&b2b);
#pragma unroll
    for (int c = 0; c < 8; ++c) sts128(row_smem + ((c ^ r7) << 4), dq_word_fast(w[c], s2, b2));
  } else {
    const float sc = qp_f32 ? __uint_as_float(sc_bits) : __uint_as_float(sc_bits << 16);
    const float bi = qp_f32 ? __uint_as_float(bi_bits) : __uint_as_float(bi_bits << 16);
#pragma unroll
    for (int c = 0; c < 8; ++c) sts128(row_smem + ((c ^ r7) << 4), dq_word_f32(w[c], sc, bi));
  }
}

// One scale or bias of the head as raw bits (see dq_store_row).
__device__ __forceinline__ uint32_t dq_load_param(const void* params, long long idx, bool qp_f32) {
  return qp_f32 ? __ldg(reinterpret_cast<const uint32_t*>(params) + idx)
                : static_cast<uint32_t>(__ldg(reinterpret_cast<const unsigned short*>(params) + idx));
}

}  // namespace b200tp
