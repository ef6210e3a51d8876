// Causal / packed-segment GQA flash attention on the Blackwell tensor cores
// (tcgen05 / TMEM / TMA), bf16 operands, head_dim 64 / 96 / 128, fp32 accumulation.
//
// Head dimension.  Every tensor-core kernel is a template on D in {64, 96, 128} (attention/api.py:44 of
// the reference: `_KERNEL_HEAD_DIMS`).  Shared-memory tiles and tensor-memory accumulators keep the
// layout of D = 128 (rows of two 64-element swizzled sub-tiles; 128 accumulator columns); what changes
// with D is the work: contractions over head_dim issue D / 16 MMA steps, products whose output is
// head_dim wide use N = D, a second sub-tile is only loaded when D > 64 (for D = 96 the tensor map's
// inner extent is 96, so TMA fills elements 96..127 with zeros), and epilogues touch D columns.  No
// padded copy of any tensor is made.
//
//   flash_fwd2_kernel  two 128-query tiles per CTA sharing every K / V tile; S and O of both
//                      tiles in tensor memory; sixteen softmax warps (two per lane quadrant and
//                      tile, half a score row each); P overwrites S columns as bf16 pairs and
//                      feeds P V as a tensor-memory operand.  Saves only O and L.
//                      On a grid smaller than the SM count with long sequences, 2-4 CTAs share
//                      each query block's key range and write un-normalised fp32 partials;
//   flash_fwd_combine_kernel  merges those partials into O and L.
//   flash_fwd_kernel   one tile per CTA, P through shared memory: taken for small grids that are
//                      not split, and selectable as a cross-check of the two-tile kernel.
//   flash_dq_kernel    one CTA per (batch, q head, 128-query block): Q and dO staged into tensor
//                      memory, S and dP = dO V^T per 64-key item in double-buffered TMEM
//                      accumulators, dS written over dP as bf16 pairs, dQ += dS K in TMEM.
//   flash_dkv_kernel   one CTA per (batch, kv head, 128-key block) walking the q heads of the GQA
//                      group in turn (or per q head when that grid would be too small), looping
//                      over the 64-query items at / below the diagonal: S^T = K Q^T and dP^T = V dO^T in TMEM
//                      (thread = key row), P^T / dS^T written back over them as bf16 pairs,
//                      dV += P^T dO and dK += dS^T Q accumulated in TMEM; bf16 output, or (per-head
//                      CTAs under GQA) fp32 partials that dkv_reduce_kernel sums over the group
//                      in a fixed order (no atomics either way: bitwise reproducible).
//
// Key blocks wholly above the diagonal or wholly in other segments are never visited
// (forward and dQ start at the block holding the first row's seg_start; dK/dV stop at the
// last query block whose first row's segment starts at or before the block's last key).
//
// Replaces attention/kernel/source.py:262-580 (forward), :863-1175 (dQ), :1430-1780
// (dK/dV) and :614-649 (D pre-pass) of the reference.
#include "flash.h"

#include <algorithm>
#include <atomic>

#include "ptx.cuh"

namespace b200tp {
namespace {

constexpr int TILE = 128;                   // queries / keys per tile
constexpr int HD = 128;                     // head_dim the tile and accumulator LAYOUTS are built for (see above)
constexpr int SUB_BYTES = TILE * 64 * 2;    // one [128 rows][64 elements] swizzled sub-tile
constexpr int TILE_BYTES = 2 * SUB_BYTES;   // 32 KiB
// Softmax / elementwise warps.  A warp can only read the TMEM lane quadrant (warp % 4), so rows
// are fixed by the quadrant and the warps of a quadrant split the COLUMNS of a block.  The
// constants below belong to the single-tile forward; the other kernels define their own.
constexpr int FWD_SPLIT = 2;                         // column parts per row in the forward
constexpr int FWD_EW_WARPS = 4 * FWD_SPLIT;
constexpr int FWD_COLS = TILE / FWD_SPLIT;           // 32 score columns and 32 head_dim columns per warp
constexpr int FWD_THREADS = 64 + 32 * FWD_EW_WARPS;
constexpr uint32_t TMEM_COLS = 512;

// ---- tile-level MMA helpers (one elected thread) ----------------------------------------
// D[128x128] (+)= A[128 x Dk] * B[128 x Dk]^T, both operands K-major, each stored as two
// [128 rows][64 k] sub-tiles; DK = contraction length (head_dim).
template <int DK>
__device__ __forceinline__ void mma_kk(uint32_t d_tmem, uint32_t a_base, uint32_t b_base, bool accumulate) {
  constexpr uint32_t idesc = make_idesc_bf16(TILE, TILE, 0, 0);
  constexpr uint32_t hi = desc_hi_sw128(1024);
  const uint32_t a_lo = desc_lo(a_base, 16), b_lo = desc_lo(b_base, 16);
#pragma unroll
  for (int kk = 0; kk < DK / 16; ++kk) {
    const uint32_t off = (kk >> 2) * SUB_BYTES + (kk & 3) * 32;
    umma_ss_w(d_tmem, a_lo + (off >> 4), hi, b_lo + (off >> 4), hi, idesc, (accumulate || kk > 0) ? 1u : 0u);
  }
}

// D[128 x DN] (+)= A[128 x 128k] * B[128k x DN]: A K-major (two [128][64k] sub-tiles), B
// MN-major: stored [128 k rows][128 n] as two sub-tiles of 64 n (each k row is 128 bytes); DN = head_dim.
template <int DN>
__device__ __forceinline__ void mma_kn(uint32_t d_tmem, uint32_t a_base, uint32_t b_base, bool accumulate) {
  constexpr uint32_t idesc = make_idesc_bf16(TILE, DN, 0, 1);
  constexpr uint32_t hi = desc_hi_sw128(1024);
  const uint32_t a_lo = desc_lo(a_base, 16), b_lo = desc_lo(b_base, SUB_BYTES);
#pragma unroll
  for (int kk = 0; kk < 8; ++kk) {
    const uint32_t a_off = (kk >> 2) * SUB_BYTES + (kk & 3) * 32;
    const uint32_t b_off = kk * 16 * 128;
    umma_ss_w(d_tmem, a_lo + (a_off >> 4), hi, b_lo + (b_off >> 4), hi, idesc, (accumulate || kk > 0) ? 1u : 0u);
  }
}

// Generic form.  A is K-major [128 rows][KTOT] in [128][64] sub-tiles, B K-major [N rows][KTOT] in
// [N][64] sub-tiles (N * 128 bytes each).
template <int N, int KTOT>
__device__ __forceinline__ void mma_kk_t(uint32_t d_tmem, uint32_t a_base, uint32_t b_base, bool accumulate) {
  constexpr uint32_t idesc = make_idesc_bf16(TILE, N, 0, 0);
  constexpr uint32_t hi = desc_hi_sw128(1024);
  const uint32_t a_lo = desc_lo(a_base, 16), b_lo = desc_lo(b_base, 16);
#pragma unroll
  for (int kk = 0; kk < KTOT / 16; ++kk) {
    const uint32_t a_off = (kk >> 2) * SUB_BYTES + (kk & 3) * 32;
    const uint32_t b_off = (kk >> 2) * (N * 128) + (kk & 3) * 32;
    umma_ss_w(d_tmem, a_lo + (a_off >> 4), hi, b_lo + (b_off >> 4), hi, idesc, (accumulate || kk > 0) ? 1u : 0u);
  }
}

// 128-row tile [128 rows][D] as [128][64] sub-tiles: the second one only when D > 64.
template <int D>
__host__ __device__ constexpr int tile_tx_bytes() { return D > 64 ? TILE_BYTES : SUB_BYTES; }
template <int D>
__device__ __forceinline__ void load_tile(uint8_t* dst, const CUtensorMap* map, uint64_t* bar, int row0, int h, int b) {
  tma_load_4d(dst, map, bar, 0, row0, h, b);
  if (D > 64) tma_load_4d(dst + SUB_BYTES, map, bar, 64, row0, h, b);
}

// 64-row tile [64 rows][D] as [64][64] sub-tiles of 8 KiB (tensor map with a 64-row box).
constexpr int HALF_TILE_BYTES = 64 * HD * 2;  // 16 KiB
template <int D>
__host__ __device__ constexpr int half_tile_tx_bytes() { return D > 64 ? HALF_TILE_BYTES : HALF_TILE_BYTES / 2; }
template <int D>
__device__ __forceinline__ void load_tile64(uint8_t* dst, const CUtensorMap* map, uint64_t* bar, int row0, int h,
                                            int b) {
  tma_load_4d(dst, map, bar, 0, row0, h, b);
  if (D > 64) tma_load_4d(dst + HALF_TILE_BYTES / 2, map, bar, 64, row0, h, b);
}

// Write 8 bf16 (one 16-byte chunk) of row `r`, element columns [8*ch, 8*ch+8) of a K-major
// swizzled [128][128] tile made of two [128][64] sub-tiles.
__device__ __forceinline__ void store_chunk(uint8_t* tile, int r, int ch, uint4 v) {
  uint8_t* p = tile + (ch >> 3) * SUB_BYTES + r * 128 + (((ch & 7) ^ (r & 7)) << 4);
  *reinterpret_cast<uint4*>(p) = v;
}

// N consecutive 32-bit TMEM columns of this thread's lane (N = 16 or a multiple of 32); no wait.
template <int N>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&v)[N]) {
  static_assert(N == 16 || N % 32 == 0, "16 columns or whole 32-column chunks");
  if constexpr (N == 16) {
    tmem_ld_x16(taddr, v);
  } else {
#pragma unroll
    for (int c = 0; c < N / 32; ++c) tmem_ld_x32(taddr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&v[c * 32]));
  }
}
template <int N>
__device__ __forceinline__ void tmem_st_cols(uint32_t taddr, const uint32_t (&v)[N]) {
  static_assert(N == 8 || N == 16 || N == 32, "8, 16 or 32 columns");
  if constexpr (N == 8) tmem_st_x8(taddr, v);
  else if constexpr (N == 16) tmem_st_x16(taddr, v);
  else tmem_st_x32(taddr, v);
}

__device__ __forceinline__ void raise(int* abort_flag, int* status, int code) {
  atomicExch(abort_flag, 1);
  if (status != nullptr) atomicCAS(status, 0, code);
}

#ifdef B200TP_TRACE
__device__ long long g_trace[16384];
#define TRACE(slot) do { if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (slot) < 16384) g_trace[(slot)] = clock64(); } while (0)
#else
#define TRACE(slot) do { } while (0)
#endif

struct AttnParams {
  int B, Hq, Hkv, S;
  float scale, scale_log2;
  const int* seg_id;
  const int* seg_start;
  // forward / dq outputs
  __nv_bfloat16* out;       // O or dQ
  long long out_sb, out_sh, out_ss;
  float* lse_out;           // forward only
  const float* lse;         // backward
  const __nv_bfloat16* o_saved;   // dQ kernel: the forward's O (same strides as dO), for D = rowsum(dO * O)
  // The row statistics of the backward (-D, -L / scale) as a bf16 operand tile for the dK / dV kernel, which
  // adds them to its products with one extra K = 16 MMA step each (see `stat_row`): per (b, q head)
  // `stat_blocks` blocks of 64 rows, each block 2048 bytes = [2 chunks][64 rows][8 bf16], the shared-memory
  // image of an unswizzled K-major tile.
  __nv_bfloat16* stat_w;          // written by the dQ kernel (or the stand-alone pre-pass)
  const __nv_bfloat16* stat;      // read by the dK / dV kernel
  int stat_blocks;
  // dkv outputs
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  long long dk_sb, dk_sh, dk_ss;
  long long dv_sb, dv_sh, dv_ss;
  float* dk_part;           // fp32 per-q-head partials (B, Hq, S, 128), null when Hq == Hkv
  float* dv_part;
  // forward split over keys (two-tile kernel, head-pair mode): grid.z = nsplit CTAs share a query block's
  // key range; each writes its un-normalised O (fp32) and (running max, row sum), combined afterwards
  int dkv_heads;            // q heads one dK / dV CTA covers: 1, or the whole GQA group (no partials then)
  int nsplit;
  int split_min;            // a query block gets min(nsplit, ceil(key blocks / split_min)) shares
  float* o_part;            // (B, Hq, nsplit, S, 128)
  float* ml_part;           // (B, Hq, nsplit, S, 2): max (log2 units, scaled scores) and row sum
  int* status;
};

__device__ __forceinline__ uint8_t* align1024(uint8_t* raw) {
  const uint32_t addr = smem_u32(raw);
  return raw + (((addr + 1023u) & ~1023u) - addr);
}

// One query row's entry of the statistics tile: -L / scale and -D, each split into three bf16 terms whose
// sum is the fp32 value exactly (each remainder is formed exactly in fp32), then two zeros:
//   [v_hi, v_mid, v_lo, d_hi, d_mid, d_lo, 0, 0].
// The dK / dV kernel multiplies the tile by constant tiles of ones (columns 0-2, or 3-5) on the tensor
// core, so S^T arrives as (K Q^T - L / scale) and dP^T as (V dO^T - D) without any per-query scalar
// reaching the elementwise warps.
__device__ __forceinline__ uint32_t bf16_bits(float x) { return __bfloat16_as_ushort(__float2bfloat16_rn(x)); }
__device__ __forceinline__ float bf16_back(uint32_t b) { return __uint_as_float(b << 16); }
__device__ __forceinline__ uint4 stat_row(float v, float d) {
  const uint32_t vh = bf16_bits(v);
  float r = v - bf16_back(vh);
  const uint32_t vm = bf16_bits(r);
  r -= bf16_back(vm);
  const uint32_t vl = bf16_bits(r);
  const uint32_t dh = bf16_bits(d);
  float q = d - bf16_back(dh);
  const uint32_t dm = bf16_bits(q);
  q -= bf16_back(dm);
  const uint32_t dl = bf16_bits(q);
  return make_uint4(vh | (vm << 16), vl | (dh << 16), dm | (dl << 16), 0u);
}
__device__ __forceinline__ void stat_store(__nv_bfloat16* stat, int stat_blocks, long long bh, int row, bool valid,
                                           float v, float d) {
  __nv_bfloat16* dst = stat + ((bh * stat_blocks + (row >> 6)) * 1024 + (row & 63) * 8);
  *reinterpret_cast<uint4*>(dst) = valid ? stat_row(v, d) : make_uint4(0u, 0u, 0u, 0u);
  *reinterpret_cast<uint4*>(dst + 512) = make_uint4(0u, 0u, 0u, 0u);
}

// =========================================================================================
// forward
// =========================================================================================
// Shared memory: Q | ring of three 128-row tiles (K_0, V_0, K_1, V_1, ... in load order) |
// P[2].  Tensor memory: S[2] (128 columns each) | O_blk[2].  S, P and O_blk are all
// double-buffered, so block n+1's softmax runs while block n's P V is on the tensor pipe.
constexpr int FWD_RING = 3;
constexpr int FWD_XCHG_BYTES = 2 * FWD_SPLIT * TILE * 4;  // [iteration parity][column part][row] partial maxima / sums
constexpr int FWD_SMEM_BYTES = (1 + FWD_RING + 2) * TILE_BYTES + 256 + FWD_XCHG_BYTES + 1024;

template <int D>
__global__ void __launch_bounds__(FWD_THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const AttnParams p) {
  griddep_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = align1024(smem_raw);
  uint8_t* q_sm = sm;
  uint8_t* ring_sm = sm + TILE_BYTES;
  uint8_t* p_sm = sm + (1 + FWD_RING) * TILE_BYTES;  // [2]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + (1 + FWD_RING + 2) * TILE_BYTES);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;    // [3]
  uint64_t* kv_empty = bars + 4;   // [3]
  uint64_t* s_full = bars + 7;     // [2]
  uint64_t* s_empty = bars + 9;    // [2]
  uint64_t* p_full = bars + 11;    // [2]
  uint64_t* o_full = bars + 13;    // [2]
  uint64_t* xch_bar = bars + 15;   // [4] one per lane quadrant: the two warps sharing its rows
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(bars + 19);
  int* abort_flag = reinterpret_cast<int*>(tmem_ptr + 1);
  float* xchg = reinterpret_cast<float*>(sm + (1 + FWD_RING + 2) * TILE_BYTES + 256);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // grid (heads x batch, query blocks): the block index is the slow one, so every head's heaviest
  // blocks are dispatched before any light one
  const int qi = gridDim.y - 1 - blockIdx.y;
  const int h = blockIdx.x % p.Hq, b = blockIdx.x / p.Hq;
  const int kvh = h / (p.Hq / p.Hkv);
  const int q0 = qi * TILE;
  const bool packed = p.seg_id != nullptr;
  const int* segs = packed ? p.seg_id + static_cast<long long>(b) * p.S : nullptr;
  int jlo = 0;
  if (packed) {
    griddep_wait();   // the segment tables may come from the kernel before this one
    int st = p.seg_start[static_cast<long long>(b) * p.S + q0];
    st = max(0, min(st, q0));
    jlo = st / TILE;
  }
  const int nblk = qi - jlo + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < FWD_RING; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], FWD_EW_WARPS);
      mbar_init(&p_full[s], FWD_EW_WARPS);
      mbar_init(&o_full[s], 1);
    }
    for (int s = 0; s < 4; ++s) mbar_init(&xch_bar[s], 32 * FWD_SPLIT);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_ptr, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_ptr);
  const uint32_t tm_o = tmem_base + 256;  // O_blk[buf] at tm_o + buf * 128; S[buf] at tmem_base + buf * 128
  griddep_wait();

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmap_q);
      tma_prefetch_desc(&tmap_k);
      tma_prefetch_desc(&tmap_v);
      mbar_arrive_expect_tx(q_full, tile_tx_bytes<D>());
      load_tile<D>(q_sm, &tmap_q, q_full, q0, h, b);
      int issued = 0;
      bool ok = true;
      for (int idx = 0; idx < 2 * nblk; ++idx) {  // even: K of block idx/2, odd: V
        const int slot = idx % FWD_RING;
        if (!mbar_wait(&kv_empty[slot], ((idx / FWD_RING) & 1) ^ 1, abort_flag)) {
          raise(abort_flag, p.status, kDevTimeoutProducer);
          ok = false;
          break;
        }
        mbar_arrive_expect_tx(&kv_full[slot], tile_tx_bytes<D>());
        load_tile<D>(ring_sm + slot * TILE_BYTES, (idx & 1) ? &tmap_v : &tmap_k, &kv_full[slot],
                     (jlo + (idx >> 1)) * TILE, kvh, b);
        ++issued;
      }
      if (!ok) {
        mbar_wait_drain(q_full, 0);
        for (int idx = max(0, issued - FWD_RING); idx < issued; ++idx)
          mbar_wait_drain(&kv_full[idx % FWD_RING], (idx / FWD_RING) & 1);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t q_a = smem_u32(q_sm), p_a = smem_u32(p_sm), ring_a = smem_u32(ring_sm);
      bool ok = mbar_wait(q_full, 0, abort_flag);
      auto issue_s = [&](int n) -> bool {
        const int idx = 2 * n, slot = idx % FWD_RING, buf = n & 1;
        if (!mbar_wait(&kv_full[slot], (idx / FWD_RING) & 1, abort_flag)) return false;
        if (!mbar_wait(&s_empty[buf], ((n >> 1) & 1) ^ 1, abort_flag)) return false;
        tc_fence_after_sync();
        mma_kk<D>(tmem_base + buf * 128, q_a, ring_a + slot * TILE_BYTES, false);
        umma_commit(&s_full[buf]);
        umma_commit(&kv_empty[slot]);  // K tile is free once S has been computed
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int n = 0; n < nblk && ok; ++n) {
        if (n + 1 < nblk) {
          ok = issue_s(n + 1);
          if (!ok) break;
        }
        const int idx = 2 * n + 1, slot = idx % FWD_RING, buf = n & 1;
        ok = mbar_wait(&p_full[buf], (n >> 1) & 1, abort_flag) &&
             mbar_wait(&kv_full[slot], (idx / FWD_RING) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
        mma_kn<D>(tm_o + buf * 128, p_a + buf * TILE_BYTES, ring_a + slot * TILE_BYTES, false);
        umma_commit(&o_full[buf]);
        umma_commit(&kv_empty[slot]);
      }
      if (!ok) raise(abort_flag, p.status, kDevTimeoutMma);
    }
  } else {
    const int quad = warp & 3;
    const int part = (warp - 2) >> 2;  // which 32 columns of S (keys) and of O (head_dim) this warp owns
    const int r = quad * 32 + lane;
    const int ig = q0 + r;
    const int igc = min(ig, p.S - 1);  // rows past the end mask like the last row; never stored
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const int my_seg = packed ? segs[igc] : 0;
    const int q_last = min(q0 + TILE - 1, p.S - 1);
    float m = -INFINITY, l = 0.f, alpha_prev = 1.f;
    float acc[FWD_COLS];
#pragma unroll
    for (int e = 0; e < FWD_COLS; ++e) acc[e] = 0.f;
    bool ok = true;
    for (int n = 0; n < nblk; ++n) {
      const int j = jlo + n;
      const int buf = n & 1;
      if (!mbar_wait_warp(&s_full[buf], (n >> 1) & 1, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      bool need_mask = (j == qi);
      if (packed) {
        const int k_first = j * TILE, k_last = min(j * TILE + TILE - 1, p.S - 1);
        const int sid = segs[k_first];
        need_mask = need_mask || sid != segs[k_last] || sid != segs[q0] || sid != segs[q_last];
      }
      // ---- this warp's 32 scores of the row, read from tensor memory once
      uint32_t sv[FWD_COLS];
      tmem_ld_cols<FWD_COLS>(tmem_base + buf * 128 + lane_off + part * FWD_COLS, sv);
      tmem_wait_ld();
      if (need_mask) {
#pragma unroll
        for (int e = 0; e < FWD_COLS; ++e) {
          const int jg = j * TILE + part * FWD_COLS + e;
          bool allowed = jg <= igc;
          if (packed && allowed) allowed = segs[jg] == my_seg;
          if (!allowed) sv[e] = 0xff800000u;  // -inf
        }
      }
      // ---- partial row max (raw scores; scale > 0 so max commutes with the scaling)
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int e = 0; e < FWD_COLS; ++e) mx4[e & 3] = fmaxf(mx4[e & 3], __uint_as_float(sv[e]));
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // ---- publish the partial max for the other threads owning this row ...
      float* slot = xchg + (n & 1) * FWD_SPLIT * TILE;
      slot[part * TILE + r] = mx;
      mbar_arrive(&xch_bar[quad]);
      // ---- ... and meanwhile fold the PREVIOUS block's P V (this warp's 32 head_dim columns)
      // into the numerator:  R_{n-1} = R_{n-2} * alpha_{n-1} + O_{n-1}
      if (n > 0) {
        const int pb = (n - 1) & 1;
        if (!mbar_wait_warp(&o_full[pb], ((n - 1) >> 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        uint32_t ov[FWD_COLS];
        tmem_ld_cols<FWD_COLS>(tm_o + pb * 128 + lane_off + part * FWD_COLS, ov);
        tmem_wait_ld();
        tmem_regs_ready(ov);
#pragma unroll
        for (int e = 0; e < FWD_COLS; ++e)
          if (part * FWD_COLS + e < D) acc[e] = fmaf(acc[e], alpha_prev, __uint_as_float(ov[e]));
      }
      if (!mbar_wait_warp(&xch_bar[quad], n & 1, abort_flag)) { ok = false; break; }
#pragma unroll
      for (int q2 = 0; q2 < FWD_SPLIT; ++q2) mx = fmaxf(mx, slot[q2 * TILE + r]);
      const float m_new = fmaxf(m, mx * p.scale_log2);
      const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = fast_exp2(m - m_safe);
      // ---- P = exp2(s - m) (masked scores are -inf -> 0), partial row sum, bf16 tile to shared
      // memory.  P[buf] is free: the fold of block n-2 waited for its P V to finish.
      uint8_t* p_tile = p_sm + buf * TILE_BYTES;
      float rs4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int g = 0; g < FWD_COLS / 8; ++g) {
        float pe[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          pe[e] = fast_exp2(fmaf(__uint_as_float(sv[g * 8 + e]), p.scale_log2, -m_safe));
          rs4[e & 3] += pe[e];
        }
        store_chunk(p_tile, r, part * (FWD_COLS / 8) + g,
                    make_uint4(pack_bf16x2(pe[0], pe[1]), pack_bf16x2(pe[2], pe[3]), pack_bf16x2(pe[4], pe[5]),
                               pack_bf16x2(pe[6], pe[7])));
      }
      l = l * alpha + ((rs4[0] + rs4[1]) + (rs4[2] + rs4[3]));  // partial: this warp's columns only
      m = m_new;
      tc_fence_before_sync();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&s_empty[buf]);
        mbar_arrive(&p_full[buf]);
      }
      alpha_prev = alpha;
    }
    const int lb = (nblk - 1) & 1;
    if (ok) ok = mbar_wait_warp(&o_full[lb], ((nblk - 1) >> 1) & 1, abort_flag);
    if (ok) {
      // all parts followed the same max sequence, so the row sum is the sum of the partials
      float* slot = xchg + (nblk & 1) * FWD_SPLIT * TILE;
      slot[part * TILE + r] = l;
      mbar_arrive(&xch_bar[quad]);
      ok = mbar_wait_warp(&xch_bar[quad], nblk & 1, abort_flag);
      if (ok) {
        l = 0.f;
#pragma unroll
        for (int q2 = 0; q2 < FWD_SPLIT; ++q2) l += slot[q2 * TILE + r];
      }
    }
    if (ok) {
      tc_fence_after_sync();
      const float inv = 1.f / l;
      __nv_bfloat16* orow =
          p.out + b * p.out_sb + h * p.out_sh + static_cast<long long>(ig) * p.out_ss + part * FWD_COLS;
      uint32_t v[FWD_COLS];
      tmem_ld_cols<FWD_COLS>(tm_o + lb * 128 + lane_off + part * FWD_COLS, v);
      tmem_wait_ld();
      if (ig < p.S) {
#pragma unroll
        for (int g = 0; g < FWD_COLS / 8; ++g) {
          if (part * FWD_COLS + g * 8 >= D) break;   // head_dim columns only
          float o8[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) o8[e] = fmaf(acc[g * 8 + e], alpha_prev, __uint_as_float(v[g * 8 + e])) * inv;
          *reinterpret_cast<uint4*>(orow + g * 8) = make_uint4(pack_bf16x2(o8[0], o8[1]), pack_bf16x2(o8[2], o8[3]),
                                                               pack_bf16x2(o8[4], o8[5]), pack_bf16x2(o8[6], o8[7]));
        }
      }
      if (ig < p.S && part == 0)
        p.lse_out[(static_cast<long long>(b) * p.Hq + h) * p.S + ig] = (m + log2f(l)) * kLn2;
    } else {
      raise(abort_flag, p.status, kDevTimeoutEpilogue);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// =========================================================================================
// forward, two query tiles per CTA
// =========================================================================================
// Two 128-query tiles share every K / V tile that is loaded: either two query heads of one GQA
// group at the same query block (even group sizes), or two consecutive query blocks of one
// head.  Each tile has its own four softmax warps with ONE THREAD PER ROW (the whole 128-score
// row lives in registers: no cross-thread reduction) and its own S and O accumulators in tensor
// memory.  P never touches shared memory: the probabilities overwrite, as bf16 pairs, part of the
// S columns they were computed from, and P V reads its A operand from there.  Per tile the
// chain S(j) -> softmax(j) -> P V(j) -> S(j+1) is serial (S(j+1) overwrites P(j), and one thread
// issues both, in order); the two tiles run half a period apart, so the tensor pipe works for one
// tile while the other is in its exp phase.  Shared memory holds only Q[2] and a four-slot ring
// of K / V tiles.
//
// O accumulates in tensor memory across key blocks (P V issued with accumulate).  The running
// max is only raised when the new block max exceeds it by more than kRescaleSlack (in log2
// units): P = exp2(s - m_used) then stays below 2^slack, row sum and O stay consistent with
// m_used, and the O rescale (TMEM load, multiply, store) happens on the rare block where the
// max really moves.  The final O / l and L = m_used ln2 + ln(l) are exact whatever m_used is.
//
// Tensor memory: S/P[2] (128 columns each) | O[2] (128 each) = 512 columns.
// Softmax warps: per tile, two warps per TMEM lane quadrant; each thread owns one row and HALF of
// its 128 score columns (and, for rescales and the epilogue, half of the 128 O columns).  Halving
// the columns per thread halves the latency of the softmax stage, which sits on the serial chain
// of its tile.  The two warps of a row exchange their block maxima (and, once, their row sums)
// through shared memory with a two-arrival mbarrier; that exchange also orders "both have loaded
// their S values" before either overwrites S columns with P.
constexpr int FWD2_SM_WARPS = 16;
constexpr int FWD2_THREADS = 64 + 32 * FWD2_SM_WARPS;
constexpr int FWD2_RING = 4;
constexpr int FWD2_XCHG_BYTES = 2 * 2 * TILE * 4;       // [tile][column half][row] fp32 block maxima
constexpr int FWD2_SMEM_BYTES = (2 + FWD2_RING) * TILE_BYTES + 256 + FWD2_XCHG_BYTES + 1024;
constexpr float kRescaleSlack = 8.f;

struct Fwd2Tile {
  int q0, h, jlo, jhi, active;
};

// Shares of a query block that sees `nb` key blocks when the launch allows up to `nsplit`.
__host__ __device__ __forceinline__ int fwd_shares(int nb, int nsplit, int split_min) {
  const int by_size = (nb + split_min - 1) / split_min;
  return by_size < nsplit ? (by_size < 1 ? 1 : by_size) : nsplit;
}

// O[128 x DN] (+)= P[128 x 128 keys] * V[128 keys x DN].  P: TMEM, bf16 pairs, two pieces of 32
// columns (keys 0..63 and 64..127) that start 64 columns apart, each written by the warp that owned
// those score columns.  V: MN-major shared-memory tile, two sub-tiles of 64 head_dim columns.
template <int DN>
__device__ __forceinline__ void mma_pv(uint32_t d_tmem, uint32_t p_tmem, uint32_t v_base, bool accumulate) {
  constexpr uint32_t idesc = make_idesc_bf16(TILE, DN, 0, 1);
  constexpr uint32_t hi = desc_hi_sw128(1024);
  const uint32_t b_lo = desc_lo(v_base, SUB_BYTES);
#pragma unroll
  for (int kk = 0; kk < 8; ++kk)
    umma_ts_w(d_tmem, p_tmem + (kk >> 2) * 64 + (kk & 3) * 8, b_lo + ((kk * 2048) >> 4), hi, idesc,
              (accumulate || kk > 0) ? 1u : 0u);
}

// 18 warps: five share one scheduler's 16 K registers, so 96 per thread is the most a launch accepts
template <int D>
__global__ void __maxnreg__(96)
flash_fwd2_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                  const __grid_constant__ CUtensorMap tmap_v, const AttnParams p, const int head_pair) {
  griddep_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = align1024(smem_raw);
  uint8_t* q_sm = sm;                                   // [2]
  uint8_t* ring_sm = sm + 2 * TILE_BYTES;               // [FWD2_RING]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + (2 + FWD2_RING) * TILE_BYTES);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;                   // [FWD2_RING]
  uint64_t* kv_empty = bars + 1 + FWD2_RING;      // [FWD2_RING]
  uint64_t* s_full = bars + 1 + 2 * FWD2_RING;    // [2] per tile: S(j) is complete (and so is every earlier MMA)
  uint64_t* p_full = s_full + 2;                  // [2] per tile: P(j) is in tensor memory
  uint64_t* o_final = s_full + 4;                 // [2] per tile: the last P V is complete
  uint64_t* xb = s_full + 6;                      // [2][4] per (tile, quadrant): the row pair's exchange
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(s_full + 14);
  float* xchg = reinterpret_cast<float*>(sm + (2 + FWD2_RING) * TILE_BYTES + 256);
  int* abort_flag = reinterpret_cast<int*>(tmem_ptr + 1);

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;   // provably warp-uniform
  // grid (head slots x batch, query block slots): the block index is the slow one, so every head's
  // heaviest blocks are dispatched before any light one
  const int hslots = head_pair ? p.Hq / 2 : p.Hq;
  const int hslot = blockIdx.x % hslots, b = blockIdx.x / hslots;
  const int nqb = (p.S + TILE - 1) / TILE;
  const bool packed = p.seg_id != nullptr;
  const int* segs = packed ? p.seg_id + static_cast<long long>(b) * p.S : nullptr;

  // ---- the two tiles of this CTA (heaviest query blocks first)
  // with a split over keys the grid is (head slots x batch, shares, query block slots), so the shares of
  // the heaviest block are still dispatched before any lighter block
  const int yslot = p.nsplit > 1 ? blockIdx.z : blockIdx.y, ny = p.nsplit > 1 ? gridDim.z : gridDim.y;
  Fwd2Tile tl[2];
  if (head_pair) {
    const int qi = ny - 1 - yslot;
    for (int t = 0; t < 2; ++t) tl[t] = {qi * TILE, 2 * hslot + t, 0, qi, 1};
  } else {
    const int pi = ny - 1 - yslot;
    for (int t = 0; t < 2; ++t) {
      const int qi = 2 * pi + t;
      tl[t] = {qi * TILE, hslot, 0, qi, qi < nqb ? 1 : 0};
    }
  }
  if (packed) griddep_wait();   // the segment tables may come from the kernel before this one
  for (int t = 0; t < 2; ++t) {
    if (packed && tl[t].active) {
      int st = p.seg_start[static_cast<long long>(b) * p.S + tl[t].q0];
      st = max(0, min(st, tl[t].q0));
      tl[t].jlo = st / TILE;
    }
  }
  // split over keys (head-pair mode only: both tiles have the same range): this CTA's share of it.  A
  // share can be empty (fewer key blocks than splits); such a CTA only writes empty partials.
  // Blocks with few key blocks are not worth splitting: they keep one share, which writes O and L
  // itself, and the CTAs of their other shares leave at once.
  const int sp = p.nsplit > 1 ? blockIdx.y : 0;
  bool cta_empty = false, partial_out = false;
  if (p.nsplit > 1) {
    const int nb = tl[0].jhi - tl[0].jlo + 1;
    const int shares = fwd_shares(nb, p.nsplit, p.split_min);
    if (sp >= shares) return;
    partial_out = shares > 1;
    if (partial_out) {
      const int per = (nb + shares - 1) / shares;
      const int lo = tl[0].jlo + sp * per, hi = min(tl[0].jhi, lo + per - 1);
      cta_empty = lo > hi;
      for (int t = 0; t < 2; ++t) {
        tl[t].jlo = lo;
        tl[t].jhi = hi;
      }
    }
  }
  const int kvh = tl[0].h / (p.Hq / p.Hkv);   // both tiles share the kv head
  const int jmin = tl[1].active ? min(tl[0].jlo, tl[1].jlo) : tl[0].jlo;
  const int jmax = tl[1].active ? max(tl[0].jhi, tl[1].jhi) : tl[0].jhi;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < FWD2_RING; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&s_full[t], 1);
      mbar_init(&p_full[t], 8);
      mbar_init(&o_final[t], 1);
      for (int q = 0; q < 4; ++q) mbar_init(&xb[t * 4 + q], 2);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_ptr, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_ptr);
  griddep_wait();

  if (warp == 0) {
    if (lane == 0 && !cta_empty) {
      tma_prefetch_desc(&tmap_q);
      tma_prefetch_desc(&tmap_k);
      tma_prefetch_desc(&tmap_v);
      mbar_arrive_expect_tx(q_full, (tl[1].active ? 2 : 1) * tile_tx_bytes<D>());
      load_tile<D>(q_sm, &tmap_q, q_full, tl[0].q0, tl[0].h, b);
      if (tl[1].active) load_tile<D>(q_sm + TILE_BYTES, &tmap_q, q_full, tl[1].q0, tl[1].h, b);
      int issued = 0;
      bool ok = true;
      const int total = 2 * (jmax - jmin + 1);
      for (int idx = 0; idx < total; ++idx) {  // even: K of block jmin + idx/2, odd: its V
        const int slot = idx % FWD2_RING;
        if (!mbar_wait(&kv_empty[slot], ((idx / FWD2_RING) & 1) ^ 1, abort_flag)) {
          raise(abort_flag, p.status, kDevTimeoutProducer);
          ok = false;
          break;
        }
        mbar_arrive_expect_tx(&kv_full[slot], tile_tx_bytes<D>());
        load_tile<D>(ring_sm + slot * TILE_BYTES, (idx & 1) ? &tmap_v : &tmap_k, &kv_full[slot],
                     (jmin + (idx >> 1)) * TILE, kvh, b);
        ++issued;
      }
      if (!ok) {
        mbar_wait_drain(q_full, 0);
        for (int idx = max(0, issued - FWD2_RING); idx < issued; ++idx)
          mbar_wait_drain(&kv_full[idx % FWD2_RING], (idx / FWD2_RING) & 1);
      }
    }
  } else if (warp == 1) {
    // The whole warp runs the issue loop (so its address arithmetic stays warp-uniform) and one
    // elected lane issues the MMAs and commits.  Step j: for each tile, P V of block j-1 (once its
    // P is in tensor memory), then S of block j, which overwrites that P.
    const uint32_t q_a = smem_u32(q_sm), ring_a = smem_u32(ring_sm);
    int np[2] = {0, 0};  // P V blocks issued so far per tile
    bool ok = cta_empty || mbar_wait_warp(q_full, 0, abort_flag);
    for (int j = jmin; j <= jmax + 1 && ok && !cta_empty; ++j) {
      const int k_idx = 2 * (j - jmin), v_idx = 2 * (j - 1 - jmin) + 1;   // ring sequence numbers
      const int k_slot = k_idx % FWD2_RING, v_slot = (v_idx + FWD2_RING) % FWD2_RING;
      if (j <= jmax) ok = mbar_wait_warp(&kv_full[k_slot], (k_idx / FWD2_RING) & 1, abort_flag);
      if (ok && j > jmin) ok = mbar_wait_warp(&kv_full[v_slot], (v_idx / FWD2_RING) & 1, abort_flag);
      for (int t = 0; t < 2 && ok; ++t) {
        if (!tl[t].active) continue;
        const bool has_prev = j - 1 >= tl[t].jlo && j - 1 <= tl[t].jhi;
        const bool has_cur = j >= tl[t].jlo && j <= tl[t].jhi;
        if (has_prev) {
          ok = mbar_wait_warp(&p_full[t], np[t] & 1, abort_flag);
          if (!ok) break;
        }
        tc_fence_after_sync();
        if (elect_one()) {
          if (has_prev) {
            mma_pv<D>(tmem_base + 256 + t * 128, tmem_base + t * 128, ring_a + v_slot * TILE_BYTES, np[t] > 0);
            if (j - 1 == tl[t].jhi) umma_commit(&o_final[t]);
          }
          if (has_cur) {
            mma_kk<D>(tmem_base + t * 128, q_a + t * TILE_BYTES, ring_a + k_slot * TILE_BYTES, false);
            umma_commit(&s_full[t]);
          }
        }
        __syncwarp();
        if (has_prev) ++np[t];
      }
      if (ok && elect_one()) {
        if (j <= jmax) umma_commit(&kv_empty[k_slot]);
        if (j > jmin) umma_commit(&kv_empty[v_slot]);
      }
      __syncwarp();
    }
    if (!ok && lane == 0) raise(abort_flag, p.status, kDevTimeoutMma);
  } else {
    const int sw = warp - 2;
    const int t = sw >> 3;           // tile of this warp
    const int ch = (sw >> 2) & 1;    // column half: scores [ch * 64, +64) of a block, O columns [ch * 64, +64)
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const Fwd2Tile me = tl[t];
    if (me.active && cta_empty) {
      // no key block in this share: an empty partial (max -inf, sum 0, O 0)
      const int ig = me.q0 + r;
      if (ig < p.S) {
        const long long prow = ((static_cast<long long>(b) * p.Hq + me.h) * p.nsplit + sp) * p.S + ig;
        float* orow = p.o_part + prow * HD + ch * 64;
#pragma unroll
        for (int g = 0; g < 16; ++g)
          if (ch * 64 + g * 4 < D) *reinterpret_cast<uint4*>(orow + g * 4) = make_uint4(0u, 0u, 0u, 0u);
        if (ch == 0) *reinterpret_cast<float2*>(p.ml_part + prow * 2) = make_float2(-INFINITY, 0.f);
      }
    } else if (me.active) {
      const int ig = me.q0 + r;
      const int igc = min(ig, p.S - 1);
      const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
      const uint32_t tm_s = tmem_base + t * 128 + lane_off;
      const uint32_t tm_o = tmem_base + 256 + t * 128 + lane_off + ch * 64;
      uint64_t* my_xb = &xb[t * 4 + quad];
      // exchange slots: block maxima xchg[(t * 2 + half) * 128 + row] (single-buffered: a warp
      // writes block n+1's value only after its partner has arrived on p_full for block n, i.e. after
      // the partner read block n's); the final row sums go, as floats, through the start of this
      // tile's Q buffer, which nothing reads once the tile's last MMA has completed.
      auto slot = [&](int half) -> volatile float* { return xchg + (t * 2 + half) * TILE + r; };
      auto sum_slot = [&](int half) -> volatile float* {
        return reinterpret_cast<float*>(q_sm + t * TILE_BYTES) + half * TILE + r;
      };
      const int my_seg = packed ? segs[igc] : 0;
      const int q_last = min(me.q0 + TILE - 1, p.S - 1);
      const int qi = me.q0 / TILE;
      const uint64_t sc2 = f2_pack(p.scale_log2, p.scale_log2);
      float m_used = -INFINITY, l = 0.f;   // l: this thread's half of the row sum
      bool ok = true;
      int n = 0;
      for (int j = me.jlo; j <= me.jhi; ++j, ++n) {
        // S(j) complete; the commit also covers P V(j-1), so O may be rescaled below.
        if (!mbar_wait_warp(&s_full[t], n & 1, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        bool need_mask = (j == qi);
        if (packed) {
          const int k_first = j * TILE, k_last = min(j * TILE + TILE - 1, p.S - 1);
          const int sid = segs[k_first];
          need_mask = need_mask || sid != segs[k_last] || sid != segs[me.q0] || sid != segs[q_last];
        }
        // 32 of this thread's 64 scores, masked; called once per pass (the scores are read twice from
        // tensor memory rather than held in 64 registers across the exchange)
        auto load_scores = [&](int c, uint32_t (&sv)[32]) {
          tmem_ld_x32(tm_s + ch * 64 + c * 32, sv);
          tmem_wait_ld();
          if (need_mask) {
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const int jg = j * TILE + ch * 64 + c * 32 + e;
              bool allowed = jg <= igc;
              if (packed && allowed) allowed = segs[jg] == my_seg;
              if (!allowed) sv[e] = 0xff800000u;  // -inf
            }
          }
        };
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t sv[32];
          load_scores(c, sv);
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
#pragma unroll
            for (int u = 0; u < 4; ++u)
              mx4[u] = fmax3(mx4[u], __uint_as_float(sv[e + 2 * u]), __uint_as_float(sv[e + 2 * u + 1]));
          }
        }
        const float mx_half = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
        // ---- exchange the half-row maxima with the partner warp (same rows, other column half)
        *slot(ch) = mx_half;
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(my_xb);
        if (!mbar_wait_warp(my_xb, n & 1, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const float mx = fmaxf(mx_half, *slot(ch ^ 1));
        // ---- raise the running max only when it really moved; rescale O on those (rare) blocks.
        // Both warps of a row see the same mx and take the same decision.
        const bool raise_max = mx > m_used + kRescaleSlack || (m_used == -INFINITY && mx > -INFINITY);
        if (__any_sync(0xffffffffu, raise_max)) {
          float alpha = 1.f;
          if (raise_max) {
            alpha = (m_used == -INFINITY) ? 0.f : fast_exp2(m_used - mx);
            l *= alpha;
            m_used = mx;
          }
          if (n > 0) {
#pragma unroll 1
            for (int c = 0; c < 2; ++c) {
              if (ch * 64 + c * 32 >= D) break;   // this thread's O columns stop at head_dim
              uint32_t ov[32];
              tmem_ld_x32(tm_o + c * 32, ov);
              tmem_wait_ld();
              tmem_regs_ready(ov);
#pragma unroll
              for (int e = 0; e < 32; ++e) ov[e] = __float_as_uint(__uint_as_float(ov[e]) * alpha);
              tmem_st_x32(tm_o + c * 32, ov);
            }
          }
        }
        const float m_safe = (m_used == -INFINITY) ? 0.f : m_used;
        // ---- P = exp2(s - m_used) as bf16 pairs over the first 32 of this thread's own 64 S columns:
        // a chunk's P lands on columns whose scores this thread has already consumed
        const uint64_t nm2 = f2_pack(-m_safe, -m_safe);
        uint64_t rs2[4] = {0ull, 0ull, 0ull, 0ull};   // four independent (even, odd) column sums
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t sv[32];
          load_scores(c, sv);
          uint32_t pk[16];
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            float x0, x1;
            f2_unpack(f2_fma(f2_pack_bits(sv[e], sv[e + 1]), sc2, nm2), x0, x1);
            x0 = fast_exp2(x0);
            x1 = fast_exp2(x1);
            rs2[(e >> 1) & 3] = f2_add(rs2[(e >> 1) & 3], f2_pack(x0, x1));
            pk[e >> 1] = pack_bf16x2(x0, x1);
          }
          tmem_st_x16(tm_s + ch * 64 + c * 16, pk);
        }
        {
          float s0, s1;
          f2_unpack(f2_add(f2_add(rs2[0], rs2[1]), f2_add(rs2[2], rs2[3])), s0, s1);
          l += s0 + s1;
        }
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[t]);
      }
      if (ok) ok = mbar_wait_warp(&o_final[t], 0, abort_flag);
      // ---- total row sum: one more exchange
      if (ok) {
        *sum_slot(ch) = l;
        __syncwarp();
        if (lane == 0) mbar_arrive(my_xb);
        ok = mbar_wait_warp(my_xb, n & 1, abort_flag);
        if (ok) l += *sum_slot(ch ^ 1);
      }
      if (ok && partial_out) {
        // this share's un-normalised O and its (max, sum); flash_fwd_combine_kernel finishes the rows
        tc_fence_after_sync();
        const long long prow = ((static_cast<long long>(b) * p.Hq + me.h) * p.nsplit + sp) * p.S + ig;
        float* orow = p.o_part + prow * HD + ch * 64;
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          if (ch * 64 + c * 32 >= D) break;
          uint32_t v[32];
          tmem_ld_x32(tm_o + c * 32, v);
          tmem_wait_ld();
          tmem_regs_ready(v);
          if (ig < p.S) {
#pragma unroll
            for (int g = 0; g < 8; ++g)
              *reinterpret_cast<uint4*>(orow + c * 32 + g * 4) = make_uint4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
          }
        }
        if (ig < p.S && ch == 0) *reinterpret_cast<float2*>(p.ml_part + prow * 2) = make_float2(m_used, l);
      } else if (ok) {
        tc_fence_after_sync();
        const float inv = 1.f / l;
        __nv_bfloat16* orow =
            p.out + b * p.out_sb + me.h * p.out_sh + static_cast<long long>(ig) * p.out_ss + ch * 64;
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          if (ch * 64 + c * 32 >= D) break;
          uint32_t v[32];
          tmem_ld_x32(tm_o + c * 32, v);
          tmem_wait_ld();
          tmem_regs_ready(v);
          if (ig < p.S) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = make_uint4(
                  pack_bf16x2(__uint_as_float(v[g * 8]) * inv, __uint_as_float(v[g * 8 + 1]) * inv),
                  pack_bf16x2(__uint_as_float(v[g * 8 + 2]) * inv, __uint_as_float(v[g * 8 + 3]) * inv),
                  pack_bf16x2(__uint_as_float(v[g * 8 + 4]) * inv, __uint_as_float(v[g * 8 + 5]) * inv),
                  pack_bf16x2(__uint_as_float(v[g * 8 + 6]) * inv, __uint_as_float(v[g * 8 + 7]) * inv));
            }
          }
        }
        if (ig < p.S && ch == 0)
          p.lse_out[(static_cast<long long>(b) * p.Hq + me.h) * p.S + ig] = (m_used + log2f(l)) * kLn2;
      } else {
        raise(abort_flag, p.status, kDevTimeoutEpilogue);
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Rows of a forward that was split over keys: O = sum_i w_i O_i / sum_i w_i l_i with
// w_i = exp2(m_i - max m), L = (max m + log2 of that sum) ln 2.  One warp per row, four head_dim
// columns per lane; the shares are added in index order.
__global__ void __launch_bounds__(128)
flash_fwd_combine_kernel(int S, int Hq, int d, int nsplit, int split_min, const int* __restrict__ seg_start,
                         const float* __restrict__ o_part, const float* __restrict__ ml_part,
                         __nv_bfloat16* __restrict__ out, long long sb, long long sh, long long ss,
                         float* __restrict__ lse_out) {
  griddep_launch_dependents();
  griddep_wait();
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int h = blockIdx.y, b = blockIdx.z;
  if (i >= S) return;
  // the row's query block and its share count, as the forward kernel derived them
  const int qi = i / TILE;
  int jlo = 0;
  if (seg_start != nullptr) jlo = max(0, min(seg_start[static_cast<long long>(b) * S + qi * TILE], qi * TILE)) / TILE;
  const int shares = fwd_shares(qi - jlo + 1, nsplit, split_min);
  if (shares == 1) return;   // written by the forward kernel itself
  const long long base = (static_cast<long long>(b) * Hq + h) * nsplit;
  float m = -INFINITY;
  for (int s = 0; s < shares; ++s) m = fmaxf(m, ml_part[((base + s) * S + i) * 2]);
  float lsum = 0.f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  const bool has_cols = lane * 4 < d;   // four head_dim columns per lane
  for (int s = 0; s < shares; ++s) {
    const long long prow = (base + s) * S + i;
    const float2 ml = *reinterpret_cast<const float2*>(ml_part + prow * 2);
    const float w = ml.x == -INFINITY ? 0.f : fast_exp2(ml.x - m);
    lsum = fmaf(w, ml.y, lsum);
    const float4 o = has_cols ? *reinterpret_cast<const float4*>(o_part + prow * HD + lane * 4)
                              : make_float4(0.f, 0.f, 0.f, 0.f);
    acc.x = fmaf(w, o.x, acc.x);
    acc.y = fmaf(w, o.y, acc.y);
    acc.z = fmaf(w, o.z, acc.z);
    acc.w = fmaf(w, o.w, acc.w);
  }
  const float inv = 1.f / lsum;
  __nv_bfloat16* orow = out + b * sb + h * sh + static_cast<long long>(i) * ss + lane * 4;
  if (has_cols)
    *reinterpret_cast<uint2*>(orow) = make_uint2(pack_bf16x2(acc.x * inv, acc.y * inv), pack_bf16x2(acc.z * inv, acc.w * inv));
  if (lane == 0) lse_out[(static_cast<long long>(b) * Hq + h) * S + i] = (m + log2f(lsum)) * kLn2;
}

// =========================================================================================
// dQ
// =========================================================================================
// Every MMA of this kernel takes its 128-row A operand from TENSOR memory, so shared memory only
// streams the 64-key K / V tiles (shared-memory operand bandwidth, not the tensor pipe, is what
// limits attention at head_dim 128 when both operands come from shared memory):
//   Q, dO (the CTA's 128 query rows) are written to TMEM once, as bf16 pairs;
//   S = Q K^T and dP = dO V^T land in double-buffered 64-column accumulators;
//   dS = P (dP - D) overwrites, as bf16 pairs, the columns of dP its thread just read;
//   dQ += dS K accumulates in TMEM over all key blocks.
// The row statistics of the backward are formed here too (attention/kernel/source.py:614-649 is a
// pre-pass in the reference): the two warps that stage a row's dO halves also read the matching halves
// of O, the half-row sums of dO * O meet in shared memory, and -D and -L log2(e) are used from there and
// published for the dK / dV kernel, which runs after this one.
// Tensor memory: Q 64 | dO 64 | S[2] 128 | dP[2] 128 | dQ 128 = 512 columns.
// Shared memory: a six-deep ring of (K, V) 64-row tile pairs.
constexpr int DQ_RING = 6;
constexpr int DQ_DPART_BYTES = 2 * TILE * 4;      // two half-row partial sums of D per query row
constexpr int DQ_SMEM_BYTES = DQ_RING * 2 * HALF_TILE_BYTES + 256 + DQ_DPART_BYTES + 1024;
// Elementwise warps of the dQ kernel: DQ_PARTS warps share a row's 64 columns of an item (DQ_CW each).
// Four narrow warps per scheduler overlap their TMEM round trips and fences better than two wide ones;
// the elementwise pass sits on the critical cycle of each S / dP buffer.
constexpr int DQ_EW_WARPS = 16;
constexpr int DQ_PARTS = DQ_EW_WARPS / 4;
constexpr int DQ_CW = 64 / DQ_PARTS;                  // S / dP columns per warp
constexpr int DQ_THREADS = 64 + 32 * DQ_EW_WARPS;
constexpr int DQ_OCOLS = HD / DQ_PARTS;               // dQ columns each warp writes in the epilogue
constexpr int DQ_STAGE_COLS = 128 / DQ_PARTS;         // Q | dO columns (bf16 pairs) each warp stages

// A [128 rows][KTOT] from TMEM (KTOT / 2 columns), B K-major [N rows][KTOT] in [N][64] sub-tiles.
template <int N, int KTOT>
__device__ __forceinline__ void mma_tk_t(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_base, bool accumulate) {
  constexpr uint32_t idesc = make_idesc_bf16(TILE, N, 0, 0);
  constexpr uint32_t hi = desc_hi_sw128(1024);
  const uint32_t b_lo = desc_lo(b_base, 16);
#pragma unroll
  for (int kk = 0; kk < KTOT / 16; ++kk) {
    const uint32_t b_off = (kk >> 2) * (N * 128) + (kk & 3) * 32;
    umma_ts_w(d_tmem, a_tmem + kk * 8, b_lo + (b_off >> 4), hi, idesc, (accumulate || kk > 0) ? 1u : 0u);
  }
}

// A [128 rows][64 k] from TMEM, stored as 64 / CW pieces of CW / 2 columns, CW columns apart (each
// elementwise warp writes its CW k values, as bf16 pairs, over the first half of the columns it owns);
// B MN-major [64 k rows][DN n] as sub-tiles of 64 n (DN = head_dim).
template <int CW, int DN>
__device__ __forceinline__ void mma_pieces_n(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_base, bool accumulate) {
  constexpr uint32_t idesc = make_idesc_bf16(TILE, DN, 0, 1);
  constexpr uint32_t hi = desc_hi_sw128(1024);
  const uint32_t b_lo = desc_lo(b_base, 64 * 128);
#pragma unroll
  for (int kk = 0; kk < 4; ++kk) {
    const int k = kk * 16;
    umma_ts_w(d_tmem, a_tmem + (k / CW) * CW + (k % CW) / 2, b_lo + ((kk * 2048) >> 4), hi, idesc,
              (accumulate || kk > 0) ? 1u : 0u);
  }
}

template <int D>
__global__ void __launch_bounds__(DQ_THREADS, 1)
flash_dq_kernel(const __grid_constant__ CUtensorMap tmap_k64, const __grid_constant__ CUtensorMap tmap_v64,
                const __nv_bfloat16* __restrict__ qg, const __nv_bfloat16* __restrict__ dog, const long long q_sb,
                const long long q_sh, const long long q_ss, const long long do_sb, const long long do_sh,
                const long long do_ss, const AttnParams p) {
  griddep_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = align1024(smem_raw);
  uint8_t* ring_sm = sm;  // stage s: K at +0, V at +16 KiB
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + DQ_RING * 2 * HALF_TILE_BYTES);
  uint64_t* kv_full = bars;                  // [6]
  uint64_t* kv_empty = bars + DQ_RING;       // [6]
  uint64_t* a_ready = bars + 2 * DQ_RING;
  uint64_t* sp_full = bars + 2 * DQ_RING + 1;   // [2]
  uint64_t* ds_full = bars + 2 * DQ_RING + 3;   // [2]
  uint64_t* dq_done = bars + 2 * DQ_RING + 5;
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(bars + 2 * DQ_RING + 6);
  int* abort_flag = reinterpret_cast<int*>(tmem_ptr + 1);
  float* dpart = reinterpret_cast<float*>(sm + DQ_RING * 2 * HALF_TILE_BYTES + 256);   // [2][TILE]

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;   // provably warp-uniform
  // grid (heads x batch, query blocks), heaviest query blocks of every head first
  const int qi = gridDim.y - 1 - blockIdx.y;
  const int h = blockIdx.x % p.Hq, b = blockIdx.x / p.Hq;
  const int kvh = h / (p.Hq / p.Hkv);
  const int q0 = qi * TILE;
  const bool packed = p.seg_id != nullptr;
  const int* segs = packed ? p.seg_id + static_cast<long long>(b) * p.S : nullptr;
  int jlo = 0;  // in 64-key blocks
  if (packed) {
    griddep_wait();   // the segment tables may come from the kernel before this one
    int st = p.seg_start[static_cast<long long>(b) * p.S + q0];
    st = max(0, min(st, q0));
    jlo = st / 64;
  }
  const int jhi = min(q0 + TILE - 1, p.S - 1) / 64;
  const int nblk = jhi - jlo + 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < DQ_RING; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(a_ready, DQ_EW_WARPS);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sp_full[s], 1);
      mbar_init(&ds_full[s], DQ_EW_WARPS);
    }
    mbar_init(dq_done, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_ptr, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_ptr);
  const uint32_t tm_q = tmem_base, tm_do = tmem_base + 64, tm_s = tmem_base + 128, tm_dp = tmem_base + 256,
                 tm_dq = tmem_base + 384;  // S / dP buffer b at + b * 64
  griddep_wait();

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmap_k64);
      tma_prefetch_desc(&tmap_v64);
      int issued = 0;
      bool ok = true;
      for (int n = 0; n < nblk; ++n) {
        const int s = n % DQ_RING;
        if (!mbar_wait(&kv_empty[s], ((n / DQ_RING) & 1) ^ 1, abort_flag)) {
          raise(abort_flag, p.status, kDevTimeoutProducer);
          ok = false;
          break;
        }
        mbar_arrive_expect_tx(&kv_full[s], 2 * half_tile_tx_bytes<D>());
        load_tile64<D>(ring_sm + s * 2 * HALF_TILE_BYTES, &tmap_k64, &kv_full[s], (jlo + n) * 64, kvh, b);
        load_tile64<D>(ring_sm + s * 2 * HALF_TILE_BYTES + HALF_TILE_BYTES, &tmap_v64, &kv_full[s], (jlo + n) * 64, kvh,
                       b);
        ++issued;
      }
      if (!ok)
        for (int n = max(0, issued - DQ_RING); n < issued; ++n) mbar_wait_drain(&kv_full[n % DQ_RING], (n / DQ_RING) & 1);
    }
  } else if (warp == 1) {
    // The whole warp runs the issue loop (so its address arithmetic stays warp-uniform) and one
    // elected lane issues the MMAs and commits.
    const uint32_t ring_a = smem_u32(ring_sm);
    bool ok = mbar_wait_warp(a_ready, 0, abort_flag);
    // S / dP buffer (n & 1) is free when block n is issued: dQ(n-2), issued earlier by the same lane,
    // is the last reader of that buffer and the tensor pipe runs one thread's MMAs in order.
    auto issue_sp = [&](int n) -> bool {
      const int s = n % DQ_RING, buf = n & 1;
      if (!mbar_wait_warp(&kv_full[s], (n / DQ_RING) & 1, abort_flag)) return false;
      tc_fence_after_sync();
      const uint32_t k_a = ring_a + s * 2 * HALF_TILE_BYTES, v_a = k_a + HALF_TILE_BYTES;
      if (elect_one()) {
        mma_tk_t<64, D>(tm_s + buf * 64, tm_q, k_a, false);     // S  = Q K^T   (128 x 64)
        mma_tk_t<64, D>(tm_dp + buf * 64, tm_do, v_a, false);   // dP = dO V^T
        umma_commit(&sp_full[buf]);
      }
      __syncwarp();
      return true;
    };
    if (ok) ok = issue_sp(0);
    for (int n = 0; n < nblk && ok; ++n) {
      if (n + 1 < nblk) {
        ok = issue_sp(n + 1);
        if (!ok) break;
      }
      const int s = n % DQ_RING, buf = n & 1;
      ok = mbar_wait_warp(&ds_full[buf], (n >> 1) & 1, abort_flag);
      if (!ok) break;
      tc_fence_after_sync();
      if (elect_one()) {
        mma_pieces_n<DQ_CW, D>(tm_dq, tm_dp + buf * 64, ring_a + s * 2 * HALF_TILE_BYTES, n > 0);  // dQ += dS K
        umma_commit(&kv_empty[s]);
        if (n == nblk - 1) umma_commit(dq_done);
      }
      __syncwarp();
    }
    if (!ok && lane == 0) raise(abort_flag, p.status, kDevTimeoutMma);
  } else {
    const int quad = warp & 3;
    const int ew = warp - 2;
    const int part = ew >> 2;          // which DQ_CW-column slice of an item this warp handles
    const int r = quad * 32 + lane;
    const int ig = q0 + r;
    const int igc = min(ig, p.S - 1);
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    // ---- stage this row's share of Q | dO (128 columns of bf16 pairs: Q at 0..63, dO at 64..127)
    // into tensor memory as the A operands
    {
      const int col0 = part * DQ_STAGE_COLS;              // first staged column
      const bool is_q = col0 < 64;
      const __nv_bfloat16* src = (is_q ? qg + b * q_sb + h * q_sh + static_cast<long long>(igc) * q_ss
                                       : dog + b * do_sb + h * do_sh + static_cast<long long>(igc) * do_ss) +
                                 (col0 & 63) * 2;
      float dsum = 0.f;   // this thread's half-row share of D = sum dO * O (dO-staging warps only)
#pragma unroll
      for (int c = 0; c < DQ_STAGE_COLS / 32; ++c) {
        uint32_t w[32];
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          uint4 v4 = make_uint4(0u, 0u, 0u, 0u);
          // elements at or past head_dim do not exist in the row (and no MMA step reads their columns)
          if (ig < p.S && (col0 & 63) * 2 + c * 64 + g * 8 < D) v4 = *reinterpret_cast<const uint4*>(src + c * 64 + g * 8);
          w[4 * g] = v4.x; w[4 * g + 1] = v4.y; w[4 * g + 2] = v4.z; w[4 * g + 3] = v4.w;
        }
        if (!is_q && ig < p.S) {
          const __nv_bfloat16* osrc =
              p.o_saved + b * do_sb + h * do_sh + static_cast<long long>(igc) * do_ss + (col0 & 63) * 2 + c * 64;
          float acc4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            if ((col0 & 63) * 2 + c * 64 + g * 8 >= D) break;
            const uint4 o4 = *reinterpret_cast<const uint4*>(osrc + g * 8);
            const uint32_t ow[4] = {o4.x, o4.y, o4.z, o4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[4 * g + e]));
              const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ow[e]));
              acc4[e] = fmaf(x.x, y.x, acc4[e]);
              acc4[e] = fmaf(x.y, y.y, acc4[e]);
            }
          }
          dsum += (acc4[0] + acc4[1]) + (acc4[2] + acc4[3]);
        }
        tmem_st_x32(tm_q + lane_off + col0 + c * 32, w);   // tm_do = tm_q + 64
      }
      if (!is_q) dpart[((col0 - 64) / DQ_STAGE_COLS) * TILE + r] = dsum;
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(a_ready);
    }
    const int my_seg = packed ? segs[igc] : 0;
    const int q_last = min(q0 + TILE - 1, p.S - 1);
    const long long ridx = (static_cast<long long>(b) * p.Hq + h) * p.S + igc;
    // -D and -L * log2(e) of this row.  All sixteen elementwise warps: the half-row sums are in shared memory
    asm volatile("bar.sync 1, %0;" ::"r"(32 * DQ_EW_WARPS) : "memory");
    const float nd = -(dpart[r] + dpart[TILE + r]);
    const float nl2 = -p.lse[ridx] * kLog2e;
    // published for the dK / dV kernel; rows past the sequence get zeros (the tile is read in whole 64-row blocks)
    if (part == 0)
      stat_store(p.stat_w, p.stat_blocks, static_cast<long long>(b) * p.Hq + h, ig, ig < p.S,
                 __fdividef(nl2, p.scale_log2), nd);
    const uint64_t sc2 = f2_pack(p.scale_log2, p.scale_log2), nl2_2 = f2_pack(nl2, nl2), nd2 = f2_pack(nd, nd);
    bool ok = true;
    for (int n = 0; n < nblk; ++n) {
      const int j = jlo + n;
      const int buf = n & 1;
      if (!mbar_wait_warp(&sp_full[buf], (n >> 1) & 1, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      const int k_first = j * 64, k_last = min(j * 64 + 63, p.S - 1);
      bool need_mask = k_first + 63 > q0;  // touches the diagonal (or runs past the sequence)
      if (packed) {
        const int sid = segs[k_first];
        need_mask = need_mask || sid != segs[k_last] || sid != segs[q0] || sid != segs[q_last];
      }
      const int c0 = part * DQ_CW;
      uint32_t sv[DQ_CW], dv[DQ_CW];
      tmem_ld_cols<DQ_CW>(tm_s + buf * 64 + lane_off + c0, sv);
      tmem_ld_cols<DQ_CW>(tm_dp + buf * 64 + lane_off + c0, dv);
      tmem_wait_ld();
      uint32_t pk[DQ_CW / 2];
#pragma unroll
      for (int e = 0; e < DQ_CW; e += 2) {
        float x0, x1;
        f2_unpack(f2_fma(f2_pack_bits(sv[e], sv[e + 1]), sc2, nl2_2), x0, x1);
        float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
        if (need_mask) {
          const int jg = k_first + c0 + e;
          bool a0 = jg <= igc, a1 = jg + 1 <= igc;
          if (packed && a0) a0 = segs[jg] == my_seg;
          if (packed && a1) a1 = segs[jg + 1] == my_seg;
          if (!a0) p0 = 0.f;
          if (!a1) p1 = 0.f;
        }
        float y0, y1;
        f2_unpack(f2_mul(f2_pack(p0, p1), f2_add(f2_pack_bits(dv[e], dv[e + 1]), nd2)), y0, y1);
        pk[e >> 1] = pack_bf16x2(y0, y1);
      }
      // dS (bf16 pairs) over the first half of the dP columns this thread has just read
      tmem_st_cols<DQ_CW / 2>(tm_dp + buf * 64 + lane_off + c0, pk);
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ds_full[buf]);
    }
    if (ok) ok = mbar_wait_warp(dq_done, 0, abort_flag);
    if (ok) {
      tc_fence_after_sync();
      __nv_bfloat16* row =
          p.out + b * p.out_sb + h * p.out_sh + static_cast<long long>(ig) * p.out_ss + part * DQ_OCOLS;
      uint32_t v[DQ_OCOLS];
      tmem_ld_cols<DQ_OCOLS>(tm_dq + lane_off + part * DQ_OCOLS, v);
      tmem_wait_ld();
      if (ig < p.S) {
#pragma unroll
        for (int g = 0; g < DQ_OCOLS / 8; ++g) {
          if (part * DQ_OCOLS + g * 8 >= D) break;
          const float s = p.scale;
          *reinterpret_cast<uint4*>(row + g * 8) = make_uint4(
              pack_bf16x2(__uint_as_float(v[g * 8]) * s, __uint_as_float(v[g * 8 + 1]) * s),
              pack_bf16x2(__uint_as_float(v[g * 8 + 2]) * s, __uint_as_float(v[g * 8 + 3]) * s),
              pack_bf16x2(__uint_as_float(v[g * 8 + 4]) * s, __uint_as_float(v[g * 8 + 5]) * s),
              pack_bf16x2(__uint_as_float(v[g * 8 + 6]) * s, __uint_as_float(v[g * 8 + 7]) * s));
        }
      }
    } else {
      raise(abort_flag, p.status, kDevTimeoutEpilogue);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// =========================================================================================
// dK / dV
// =========================================================================================
// One CTA per (128-key block, q head), or per (128-key block, GQA group) when that still gives
// about 1.7 CTAs per SM: the group's q heads then stream past the same K / V tiles one after the
// other, dK / dV accumulate over all of them in tensor memory and are written once, as bf16, with no
// fp32 partials and no reduce pass.  Query blocks of 64 stream through a ring; S^T = K Q^T and
// dP^T = V dO^T land in double-buffered 64-column TMEM accumulators (thread = key row); P^T and
// dS^T are written back, as bf16 pairs, over the columns their thread has just read, and feed
// dV += P^T dO and dK += dS^T Q as TENSOR-memory A operands (no shared-memory round trip).
// The per-query scalars of the elementwise pass (-L log2 e inside the exponential, -D beside dP) never
// reach the elementwise warps: the dQ kernel leaves them as a small bf16 tile (`stat_row`), the producer
// brings each item's 64 rows in with one bulk copy, and each issuer appends one K = 16 step to its first
// product -- A = a constant tile of ones in the three columns of its statistic, B = the statistics tile --
// so the accumulators hold K Q^T - L / scale and V dO^T - D when the elementwise warps read them.  (Read
// from shared memory as broadcast loads, the scalars took 28 % of the shared-memory pipe's cycles in a
// kernel whose tensor-core operands already take 58 %.)
// Shared memory: K | V | ring of four (Q, dO) 64-row tile pairs | per-warp segment ids | ring of statistics
// blocks | two tiles of ones.
// Tensor memory: S^T[2] 128 | dP^T[2] 128 | dV 128 | dK 128.
constexpr int DKV_RING = 4;
// Elementwise warps: DKV_PARTS warps share a key row's 64 query columns of an item (DKV_CW each); see
// the note on the dQ kernel's warps.
constexpr int DKV_EW_WARPS = 16;
constexpr int DKV_PARTS = DKV_EW_WARPS / 4;
constexpr int DKV_CW = 64 / DKV_PARTS;
constexpr int DKV_CTRL_WARPS = 3;                     // TMA producer and two MMA issuers
constexpr int DKV_THREADS = 32 * DKV_CTRL_WARPS + 32 * DKV_EW_WARPS;
constexpr int DKV_OCOLS = HD / DKV_PARTS;             // dK / dV columns each warp writes in the epilogue
constexpr int DKV_SCAL_BYTES = DKV_EW_WARPS * 32 * 4;   // per warp: the segment ids of an item's queries (packed rows)
constexpr int DKV_STAT_BYTES = 2048;                   // one 64-query block of the statistics tile
constexpr int DKV_ONES_BYTES = 4096;                   // [2 chunks][128 rows][8 bf16]: a constant A operand
constexpr int DKV_SMEM_BYTES = 2 * TILE_BYTES + DKV_RING * 2 * HALF_TILE_BYTES + 256 + DKV_SCAL_BYTES +
                               DKV_RING * DKV_STAT_BYTES + 2 * DKV_ONES_BYTES + 1024;

template <int D>
__global__ void __launch_bounds__(DKV_THREADS, 1)
flash_dkv_kernel(const __grid_constant__ CUtensorMap tmap_q64, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do64,
                 const AttnParams p) {
  griddep_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = align1024(smem_raw);
  uint8_t* k_sm = sm;
  uint8_t* v_sm = sm + TILE_BYTES;
  uint8_t* ring_sm = sm + 2 * TILE_BYTES;                        // stage s: Q at +0, dO at +16 KiB
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring_sm + DKV_RING * 2 * HALF_TILE_BYTES);
  uint8_t* scal_sm = ring_sm + DKV_RING * 2 * HALF_TILE_BYTES + 256;
  uint8_t* stat_sm = scal_sm + DKV_SCAL_BYTES;                  // [DKV_RING][2048]
  uint8_t* ones_sm = stat_sm + DKV_RING * DKV_STAT_BYTES;       // ones in columns 0-2, then ones in columns 3-5
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;                 // [DKV_RING]
  uint64_t* qdo_empty = bars + 1 + DKV_RING;     // [DKV_RING]
  uint64_t* sp_full = bars + 1 + 2 * DKV_RING;   // [2]
  uint64_t* pds_full = sp_full + 2;              // [2]
  uint64_t* acc_done = sp_full + 4;
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(sp_full + 5);
  int* abort_flag = reinterpret_cast<int*>(tmem_ptr + 1);
  int* ihi_sm = abort_flag + 1;

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;   // provably warp-uniform
  // grid (heads x batch, key blocks): key block 0 (seen by every query) of every head first
  const int jb = blockIdx.y;
  const int hslots = p.Hq / p.dkv_heads;
  const int hq_idx = (blockIdx.x % hslots) * p.dkv_heads, b = blockIdx.x / hslots;   // first q head of this CTA
  const int group = p.Hq / p.Hkv;
  const int kvh = hq_idx / group;
  const int k0 = jb * TILE;
  const bool packed = p.seg_id != nullptr;
  const int* segs = packed ? p.seg_id + static_cast<long long>(b) * p.S : nullptr;
  const int nqb = (p.S + 63) / 64;   // 64-row query blocks
  const int ilo = k0 / 64;           // first query block that can see a key of this block

  if (packed) griddep_wait();   // thread 0 reads the segment table below
  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < DKV_RING; ++s) {
      mbar_init(&qdo_full[s], 1);
      mbar_init(&qdo_empty[s], 2);   // one commit from each issuer
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sp_full[s], 2);     // S^T from one issuer, dP^T from the other
      mbar_init(&pds_full[s], DKV_EW_WARPS);
    }
    mbar_init(acc_done, 2);
    *abort_flag = 0;
    // last query block that can see any key of this block
    int ihi = nqb - 1;
    if (packed) {
      const int k_last = min(k0 + TILE - 1, p.S - 1);
      const int* starts = p.seg_start + static_cast<long long>(b) * p.S;
      ihi = ilo;
      while (ihi + 1 < nqb && starts[(ihi + 1) * 64] <= k_last) ++ihi;
    }
    *ihi_sm = ihi;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_ptr, TMEM_COLS);
    tmem_relinquish();
  }
  if (threadIdx.x < 512) {
    // two unswizzled K-major tiles [2 chunks][128 rows][8 bf16]; chunk 1 (k = 8..15) is zero
    const int tile = threadIdx.x >> 8, chunk = (threadIdx.x >> 7) & 1, row = threadIdx.x & 127;
    const uint32_t one2 = 0x3F803F80u;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (chunk == 0) val = tile == 0 ? make_uint4(one2, 0x00003F80u, 0u, 0u) : make_uint4(0u, 0x3F800000u, one2, 0u);
    *reinterpret_cast<uint4*>(ones_sm + tile * DKV_ONES_BYTES + chunk * 2048 + row * 16) = val;
    fence_proxy_async_smem();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_ptr);
  const uint32_t tm_st = tmem_base, tm_dpt = tmem_base + 128, tm_dv = tmem_base + 256, tm_dk = tmem_base + 384;
  const int ihi = *reinterpret_cast<volatile int*>(ihi_sm);
  griddep_wait();
  const int nq = ihi - ilo + 1;    // query blocks per head
  const int total = nq * p.dkv_heads;   // loop items: the 64-row query blocks of each q head of this CTA in turn

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmap_q64);
      tma_prefetch_desc(&tmap_k);
      tma_prefetch_desc(&tmap_v);
      tma_prefetch_desc(&tmap_do64);
      mbar_arrive_expect_tx(kv_full, 2 * tile_tx_bytes<D>());
      load_tile<D>(k_sm, &tmap_k, kv_full, k0, kvh, b);
      load_tile<D>(v_sm, &tmap_v, kv_full, k0, kvh, b);
      int issued = 0;
      bool ok = true;
      for (int t = 0; t < total; ++t) {
        const int hh = t / nq;
        const int h = hq_idx + hh;
        const int i = ilo + (t - hh * nq);
        const int s = t % DKV_RING;
        if (!mbar_wait(&qdo_empty[s], ((t / DKV_RING) & 1) ^ 1, abort_flag)) {
          raise(abort_flag, p.status, kDevTimeoutProducer);
          ok = false;
          break;
        }
        mbar_arrive_expect_tx(&qdo_full[s], 2 * half_tile_tx_bytes<D>() + DKV_STAT_BYTES);
        load_tile64<D>(ring_sm + s * 2 * HALF_TILE_BYTES, &tmap_q64, &qdo_full[s], i * 64, h, b);
        load_tile64<D>(ring_sm + s * 2 * HALF_TILE_BYTES + HALF_TILE_BYTES, &tmap_do64, &qdo_full[s], i * 64, h, b);
        bulk_load(stat_sm + s * DKV_STAT_BYTES,
                  p.stat + ((static_cast<long long>(b) * p.Hq + h) * p.stat_blocks + i) * 1024, DKV_STAT_BYTES,
                  &qdo_full[s]);
        ++issued;
      }
      if (!ok) {
        mbar_wait_drain(kv_full, 0);
        for (int t = max(0, issued - DKV_RING); t < issued; ++t)
          mbar_wait_drain(&qdo_full[t % DKV_RING], (t / DKV_RING) & 1);
      }
    }
  } else if (warp == 1 || warp == 2) {
    // ---- two issuers: the tensor pipe takes an N=64 MMA from a single thread only every ~46 clocks
    // (32 clocks of tensor time), and from two threads every ~34.  Issuer 1: S^T = K Q^T and
    // dV += P^T dO; issuer 2: dP^T = V dO^T and dK += dS^T Q.  Each issuer owns one of the two aliased
    // buffers: S^T(t) becomes P^T(t), read by dV(t), before S^T(t+2) overwrites it, and all three are
    // issued by the same lane, in order (likewise dP^T / dS^T / dK).  The whole warp runs the loop
    // (warp-uniform address arithmetic); one elected lane issues.
    const bool first = warp == 1;
    const uint32_t a_addr = first ? smem_u32(k_sm) : smem_u32(v_sm);
    const uint32_t ring_a = smem_u32(ring_sm);
    const uint32_t tm_in = first ? tm_st : tm_dpt;          // product of this issuer, later its A operand
    const uint32_t tm_acc = first ? tm_dv : tm_dk;
    const uint32_t b1_off = first ? 0u : HALF_TILE_BYTES;   // B of the first product: Q (S^T) or dO (dP^T)
    const uint32_t b2_off = first ? HALF_TILE_BYTES : 0u;   // B of the second: dO (dV) or Q (dK)
    // the statistics step: A = this issuer's tile of ones (chunks 2048 bytes apart), B = the item's block of
    // the statistics tile (chunks 1024 bytes apart); 8-row groups 128 bytes apart in both
    const uint32_t ones_lo = desc_lo(smem_u32(ones_sm) + (first ? 0u : DKV_ONES_BYTES), 2048);
    const uint32_t stat_a = smem_u32(stat_sm);
    bool ok = mbar_wait_warp(kv_full, 0, abort_flag);
    auto issue_in = [&](int t) -> bool {
      const int s = t % DKV_RING, buf = t & 1;
      if (!mbar_wait_warp(&qdo_full[s], (t / DKV_RING) & 1, abort_flag)) return false;
      tc_fence_after_sync();
      if (elect_one()) {
        mma_kk_t<64, D>(tm_in + buf * 64, a_addr, ring_a + s * 2 * HALF_TILE_BYTES + b1_off, false);
        umma_ss_w(tm_in + buf * 64, ones_lo, desc_hi_plain(128), desc_lo(stat_a + s * DKV_STAT_BYTES, 1024),
                  desc_hi_plain(128), make_idesc_bf16(TILE, 64, 0, 0), 1u);
        umma_commit(&sp_full[buf]);
      }
      __syncwarp();
      return true;
    };
    if (ok) ok = issue_in(0);
    for (int t = 0; t < total && ok; ++t) {
      if (t + 1 < total) {
        ok = issue_in(t + 1);
        if (!ok) break;
      }
      const int s = t % DKV_RING, buf = t & 1;
      ok = mbar_wait_warp(&pds_full[buf], (t >> 1) & 1, abort_flag);
      if (!ok) break;
      tc_fence_after_sync();
      if (elect_one()) {
        mma_pieces_n<DKV_CW, D>(tm_acc, tm_in + buf * 64, ring_a + s * 2 * HALF_TILE_BYTES + b2_off, t > 0);
        umma_commit(&qdo_empty[s]);
        if (t == total - 1) umma_commit(acc_done);
      }
      __syncwarp();
    }
    if (!ok && lane == 0) raise(abort_flag, p.status, kDevTimeoutMma);
  } else {
    const int quad = warp & 3;
    const int ew = warp - DKV_CTRL_WARPS;
    const int part = ew >> 2;              // which DKV_CW-query slice of an item this warp handles
    const int r = quad * 32 + lane;        // key row inside the block
    const int kg = k0 + r;
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const int my_seg = (packed && kg < p.S) ? segs[kg] : 0;
    // Warp-private staging of the segment ids of an item's queries (packed rows, masked items only), read
    // back as broadcast vector loads.
    int* my_sg = reinterpret_cast<int*>(scal_sm) + ew * 32;
    const uint64_t sc2 = f2_pack(p.scale_log2, p.scale_log2);
    bool ok = true;
    for (int t = 0; t < total; ++t) {
      const int hh = t / nq;
      const int i = ilo + (t - hh * nq);
      const int buf = t & 1;
      const uint32_t ph = (t >> 1) & 1;
      const int q_first = i * 64 + part * DKV_CW;
      // Warp-uniform: can any (key, query) pair of this warp's 128 x DKV_CW sub-block be masked?
      // Segment ids do not decrease along a row, so comparing the two ends covers the block.
      bool need_mask = q_first < k0 + TILE - 1 || q_first + DKV_CW - 1 >= p.S;
      if (packed && !need_mask) need_mask = segs[k0] != segs[q_first + DKV_CW - 1];
      if (packed && need_mask) {
        const int qmine = q_first + lane;
        __syncwarp();   // the previous masked item's reads of the staging area are done
        if (lane < DKV_CW) my_sg[lane] = qmine < p.S ? segs[qmine] : -1;
        __syncwarp();
      }
      if (!mbar_wait_warp(&sp_full[buf], ph, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      uint32_t sv[DKV_CW], dv[DKV_CW];
      tmem_ld_cols<DKV_CW>(tm_st + buf * 64 + lane_off + part * DKV_CW, sv);
      tmem_ld_cols<DKV_CW>(tm_dpt + buf * 64 + lane_off + part * DKV_CW, dv);
      tmem_wait_ld();
      uint32_t pk_p[DKV_CW / 2], pk_ds[DKV_CW / 2];
#pragma unroll
      for (int e = 0; e < DKV_CW; e += 2) {
        // sv = K Q^T - L / scale, dv = V dO^T - D (the statistics step of the products)
        float x0, x1;
        f2_unpack(f2_mul(f2_pack_bits(sv[e], sv[e + 1]), sc2), x0, x1);
        float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
        if (need_mask) {
          // visible iff the query exists, is at or after this key, and shares its segment
          bool a0 = kg <= q_first + e && q_first + e < p.S, a1 = kg <= q_first + e + 1 && q_first + e + 1 < p.S;
          if (packed) {
            const int2 sg = *reinterpret_cast<const int2*>(my_sg + e);
            a0 = a0 && sg.x == my_seg;
            a1 = a1 && sg.y == my_seg;
          }
          if (!a0) p0 = 0.f;
          if (!a1) p1 = 0.f;
        }
        float y0, y1;
        f2_unpack(f2_mul(f2_pack(p0, p1), f2_pack_bits(dv[e], dv[e + 1])), y0, y1);
        pk_p[e >> 1] = pack_bf16x2(p0, p1);
        pk_ds[e >> 1] = pack_bf16x2(y0, y1);
      }
      // P^T / dS^T (bf16 pairs) over the first half of the columns this thread has just read
      tmem_st_cols<DKV_CW / 2>(tm_st + buf * 64 + lane_off + part * DKV_CW, pk_p);
      tmem_st_cols<DKV_CW / 2>(tm_dpt + buf * 64 + lane_off + part * DKV_CW, pk_ds);
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&pds_full[buf]);
    }
    if (ok) ok = mbar_wait_warp(acc_done, 0, abort_flag);
    if (ok) {
      tc_fence_after_sync();
      if (p.dk_part != nullptr) {
        // GQA: this CTA covered one q head; write fp32 partials, summed over the group afterwards
        const long long prow = ((static_cast<long long>(b) * p.Hq + hq_idx) * p.S + kg) * HD + part * DKV_OCOLS;
#pragma unroll
        for (int cc = 0; cc < DKV_OCOLS / 32; ++cc) {
          if (part * DKV_OCOLS + cc * 32 >= D) break;   // head_dim columns only
          uint32_t a[32], bb[32];
          tmem_ld_x32(tm_dv + lane_off + part * DKV_OCOLS + cc * 32, a);
          tmem_ld_x32(tm_dk + lane_off + part * DKV_OCOLS + cc * 32, bb);
          tmem_wait_ld();
          tmem_regs_ready(a);
          tmem_regs_ready(bb);
          if (kg < p.S) {
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              *reinterpret_cast<uint4*>(p.dv_part + prow + cc * 32 + g * 4) =
                  make_uint4(a[g * 4], a[g * 4 + 1], a[g * 4 + 2], a[g * 4 + 3]);
              *reinterpret_cast<uint4*>(p.dk_part + prow + cc * 32 + g * 4) =
                  make_uint4(bb[g * 4], bb[g * 4 + 1], bb[g * 4 + 2], bb[g * 4 + 3]);
            }
          }
        }
      } else {
      __nv_bfloat16* dkrow =
          p.dk + b * p.dk_sb + kvh * p.dk_sh + static_cast<long long>(kg) * p.dk_ss + part * DKV_OCOLS;
      __nv_bfloat16* dvrow =
          p.dv + b * p.dv_sb + kvh * p.dv_sh + static_cast<long long>(kg) * p.dv_ss + part * DKV_OCOLS;
#pragma unroll
      for (int cc = 0; cc < DKV_OCOLS / 32; ++cc) {
        if (part * DKV_OCOLS + cc * 32 >= D) break;   // head_dim columns only
        uint32_t a[32], bb[32];
        tmem_ld_x32(tm_dv + lane_off + part * DKV_OCOLS + cc * 32, a);
        tmem_ld_x32(tm_dk + lane_off + part * DKV_OCOLS + cc * 32, bb);
        tmem_wait_ld();
        tmem_regs_ready(a);
        tmem_regs_ready(bb);
        if (kg < p.S) {
          const float s = p.scale;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            *reinterpret_cast<uint4*>(dvrow + cc * 32 + g * 8) = make_uint4(
                pack_bf16x2(__uint_as_float(a[g * 8]), __uint_as_float(a[g * 8 + 1])),
                pack_bf16x2(__uint_as_float(a[g * 8 + 2]), __uint_as_float(a[g * 8 + 3])),
                pack_bf16x2(__uint_as_float(a[g * 8 + 4]), __uint_as_float(a[g * 8 + 5])),
                pack_bf16x2(__uint_as_float(a[g * 8 + 6]), __uint_as_float(a[g * 8 + 7])));
            *reinterpret_cast<uint4*>(dkrow + cc * 32 + g * 8) = make_uint4(
                pack_bf16x2(__uint_as_float(bb[g * 8]) * s, __uint_as_float(bb[g * 8 + 1]) * s),
                pack_bf16x2(__uint_as_float(bb[g * 8 + 2]) * s, __uint_as_float(bb[g * 8 + 3]) * s),
                pack_bf16x2(__uint_as_float(bb[g * 8 + 4]) * s, __uint_as_float(bb[g * 8 + 5]) * s),
                pack_bf16x2(__uint_as_float(bb[g * 8 + 6]) * s, __uint_as_float(bb[g * 8 + 7]) * s));
          }
        }
      }
      }
    } else {
      raise(abort_flag, p.status, kDevTimeoutEpilogue);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Row statistics of the backward, one warp per row: -D = -rowsum(dO * O)
// (attention/kernel/source.py:614-649) and -L / scale, written as the statistics tile of the dK / dV
// kernel.  Only launched when the dQ kernel, which forms the same tile in its prologue, is left out.
__global__ void __launch_bounds__(128)
bwd_d_kernel(int S, int Hq, int d, const __nv_bfloat16* __restrict__ d_o, const __nv_bfloat16* __restrict__ o, long long sb,
             long long sh, long long ss, const float* __restrict__ lse, __nv_bfloat16* __restrict__ stat,
             int stat_blocks, float scale_log2) {
  griddep_launch_dependents();
  griddep_wait();
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int h = blockIdx.y, b = blockIdx.z;
  if (i >= S) {
    // the grid covers the statistics tile's whole 64-row blocks: rows past the sequence are zeros
    if (lane == 0 && i < stat_blocks * 64) stat_store(stat, stat_blocks, static_cast<long long>(b) * Hq + h, i, false, 0.f, 0.f);
    return;
  }
  const long long off = b * sb + h * sh + static_cast<long long>(i) * ss + lane * 4;
  const bool has_cols = lane * 4 < d;   // four head_dim columns per lane
  const uint2 a = has_cols ? *reinterpret_cast<const uint2*>(d_o + off) : make_uint2(0u, 0u);
  const uint2 c = has_cols ? *reinterpret_cast<const uint2*>(o + off) : make_uint2(0u, 0u);
  const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* c2 = reinterpret_cast<const __nv_bfloat162*>(&c);
  float s = 0.f;
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const float2 x = __bfloat1622float2(a2[e]), y = __bfloat1622float2(c2[e]);
    s = fmaf(x.x, y.x, s);
    s = fmaf(x.y, y.y, s);
  }
#pragma unroll
  for (int ofs = 16; ofs > 0; ofs >>= 1) s += __shfl_xor_sync(0xffffffffu, s, ofs);
  if (lane == 0) {
    const long long r = (static_cast<long long>(b) * Hq + h) * S + i;
    stat_store(stat, stat_blocks, static_cast<long long>(b) * Hq + h, i, true, __fdividef(-lse[r] * kLog2e, scale_log2), -s);
  }
}

// dK / dV = sum over the GQA group of the fp32 per-q-head partials (fixed order: bitwise
// reproducible), dK scaled, cast once.  One thread per 8 head_dim elements.
__global__ void __launch_bounds__(256)
dkv_reduce_kernel(int B, int Hq, int Hkv, int S, int d, float scale, const float* __restrict__ dk_part,
                  const float* __restrict__ dv_part, __nv_bfloat16* __restrict__ dk, __nv_bfloat16* __restrict__ dv,
                  long long dk_sb, long long dk_sh, long long dk_ss, long long dv_sb, long long dv_sh, long long dv_ss) {
  griddep_launch_dependents();
  griddep_wait();
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long total = static_cast<long long>(B) * Hkv * S * (d / 8);
  if (idx >= total) return;
  const int c8 = static_cast<int>(idx % (d / 8));
  const long long row = idx / (d / 8);
  const int srow = static_cast<int>(row % S);
  const int kvh = static_cast<int>((row / S) % Hkv);
  const int b = static_cast<int>(row / (static_cast<long long>(S) * Hkv));
  const int group = Hq / Hkv;
  float ak[8] = {0, 0, 0, 0, 0, 0, 0, 0}, av[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int g = 0; g < group; ++g) {
    const long long off = ((static_cast<long long>(b) * Hq + kvh * group + g) * S + srow) * HD + c8 * 8;
    const float4 k0 = *reinterpret_cast<const float4*>(dk_part + off), k1 = *reinterpret_cast<const float4*>(dk_part + off + 4);
    const float4 v0 = *reinterpret_cast<const float4*>(dv_part + off), v1 = *reinterpret_cast<const float4*>(dv_part + off + 4);
    ak[0] += k0.x; ak[1] += k0.y; ak[2] += k0.z; ak[3] += k0.w; ak[4] += k1.x; ak[5] += k1.y; ak[6] += k1.z; ak[7] += k1.w;
    av[0] += v0.x; av[1] += v0.y; av[2] += v0.z; av[3] += v0.w; av[4] += v1.x; av[5] += v1.y; av[6] += v1.z; av[7] += v1.w;
  }
  __nv_bfloat16* dkp = dk + b * dk_sb + kvh * dk_sh + static_cast<long long>(srow) * dk_ss + c8 * 8;
  __nv_bfloat16* dvp = dv + b * dv_sb + kvh * dv_sh + static_cast<long long>(srow) * dv_ss + c8 * 8;
  *reinterpret_cast<uint4*>(dkp) = make_uint4(pack_bf16x2(ak[0] * scale, ak[1] * scale), pack_bf16x2(ak[2] * scale, ak[3] * scale),
                                              pack_bf16x2(ak[4] * scale, ak[5] * scale), pack_bf16x2(ak[6] * scale, ak[7] * scale));
  *reinterpret_cast<uint4*>(dvp) = make_uint4(pack_bf16x2(av[0], av[1]), pack_bf16x2(av[2], av[3]),
                                              pack_bf16x2(av[4], av[5]), pack_bf16x2(av[6], av[7]));
}

int configure() {
  static std::atomic<int> done[64];
  int dev = 0;
  B200TP_CUDA_OK(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && done[dev].load(std::memory_order_acquire)) return B200TP_OK;
#define B200TP_SET_SMEM(D)                                                                                          \
  B200TP_CUDA_OK(cudaFuncSetAttribute(flash_fwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,            \
                                      FWD_SMEM_BYTES));                                                            \
  B200TP_CUDA_OK(cudaFuncSetAttribute(flash_fwd2_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,           \
                                      FWD2_SMEM_BYTES));                                                           \
  B200TP_CUDA_OK(cudaFuncSetAttribute(flash_dq_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,             \
                                      DQ_SMEM_BYTES));                                                             \
  B200TP_CUDA_OK(cudaFuncSetAttribute(flash_dkv_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,            \
                                      DKV_SMEM_BYTES));
  B200TP_SET_SMEM(64)
  B200TP_SET_SMEM(96)
  B200TP_SET_SMEM(128)
#undef B200TP_SET_SMEM
  if (dev >= 0 && dev < 64) done[dev].store(1, std::memory_order_release);
  return B200TP_OK;
}

AttnParams base_params(const b200tp_attn_args* a, int* status) {
  AttnParams p{};
  p.B = a->b; p.Hq = a->hq; p.Hkv = a->hkv; p.S = a->s;
  p.scale = a->scale;
  p.scale_log2 = a->scale * kLog2e;
  p.seg_id = a->seg_id;
  p.seg_start = a->seg_start;
  p.status = status;
  return p;
}

}  // namespace

// Number of CTAs that share a query block's key range in the forward, or 0 for no split.  A grid of
// fewer two-tile CTAs than SMs (few heads, one sequence: e.g. one kv-head group per GPU) is bound by
// the serial chain of its longest query block; splitting every block's key range shortens that chain
// and fills the SMs.  Head-pair mode only (an even GQA group).  Bits 3-5 of `reserved` force a share
// count of 2-4.
// Key blocks per share below which a query block is not split further.  1: every block with at least
// two key blocks is split (leaving the light blocks whole was measured 10-15 % slower).
constexpr int kFwdSplitMin = 1;
static int fwd_splits(const b200tp_attn_args* a) {
  const int group = a->hq / a->hkv;
  const int fwd_choice = a->reserved & 3;
  if (group % 2 != 0 || fwd_choice == 1) return 0;
  const int forced = (a->reserved >> 3) & 7;
  if (forced >= 2) return std::min(forced, 4);
  if (fwd_choice == 2) return 0;
  const int nqb = (a->s + TILE - 1) / TILE;
  const long long ctas = static_cast<long long>(a->b) * (a->hq / 2) * nqb;
  // measured: worth its partial writes and combine pass from 64 key blocks on, or from 32 when the
  // unsplit grid would not even fill half of the SMs
  if (ctas > sm_count() || nqb < 32 || (nqb < 64 && 2 * ctas > sm_count())) return 0;
  const long long want = (17LL * sm_count() + 10 * ctas - 1) / (10 * ctas);   // about 1.7 CTAs per SM
  return static_cast<int>(std::min<long long>(4, std::max<long long>(2, want)));
}

size_t flash_tc_fwd_workspace_bytes(const b200tp_attn_args* a) {
  const int ns = fwd_splits(a);
  if (ns == 0) return 0;
  const size_t rows = static_cast<size_t>(a->b) * a->hq * ns * a->s;
  return align_up(rows * HD * sizeof(float), 256) + align_up(rows * 2 * sizeof(float), 256);
}

template <int D>
static int fwd_impl(const b200tp_attn_args* a, const void* q, const void* k, const void* v, void* o, float* lse,
                    void* workspace, size_t workspace_bytes, cudaStream_t stream, int* status) {
  int rc = configure();
  if (rc) return rc;
  if (!(a->scale > 0.f)) return fail(B200TP_ERR_ATTN_INPUT, "scale must be positive");
  // the maps carry the real head_dim: a box that reaches past it is zero-filled by TMA
  CUtensorMap tq, tk, tv;
  rc = make_tmap_bhsd_bf16(&tq, q, a->b, a->hq, a->s, D, a->q_stride[0], a->q_stride[1], a->q_stride[2], TILE, 64);
  if (rc) return rc;
  rc = make_tmap_bhsd_bf16(&tk, k, a->b, a->hkv, a->s, D, a->k_stride[0], a->k_stride[1], a->k_stride[2], TILE, 64);
  if (rc) return rc;
  rc = make_tmap_bhsd_bf16(&tv, v, a->b, a->hkv, a->s, D, a->v_stride[0], a->v_stride[1], a->v_stride[2], TILE, 64);
  if (rc) return rc;
  AttnParams p = base_params(a, status);
  p.out = static_cast<__nv_bfloat16*>(o);
  p.out_sb = a->o_stride[0]; p.out_sh = a->o_stride[1]; p.out_ss = a->o_stride[2];
  p.lse_out = lse;
  const int nqb = (a->s + TILE - 1) / TILE;
  const int group = a->hq / a->hkv;
  // Two tiles per CTA halve the CTA count.  When that would leave fewer CTAs than SMs (a short
  // batch of few heads, e.g. one kv-head group per GPU), the single-tile kernel's finer work units
  // balance the causal triangle better and win.
  const long long two_tile_ctas =
      static_cast<long long>(a->b) * (group % 2 == 0 ? a->hq / 2 * nqb : a->hq * ((nqb + 1) / 2));
  const size_t ws_need = flash_tc_fwd_workspace_bytes(a);
  if (ws_need != 0 && workspace != nullptr && workspace_bytes >= ws_need) {
    // split over keys: partials from the two-tile kernel, then one combine pass
    const int ns = fwd_splits(a);
    const size_t rows = static_cast<size_t>(a->b) * a->hq * ns * a->s;
    p.nsplit = ns;
    p.split_min = kFwdSplitMin;
    p.o_part = static_cast<float*>(workspace);
    p.ml_part = reinterpret_cast<float*>(static_cast<char*>(workspace) + align_up(rows * HD * sizeof(float), 256));
    dim3 grid(a->hq / 2 * a->b, ns, nqb);
    B200TP_CUDA_OK(launch_pdl(flash_fwd2_kernel<D>, grid, dim3(FWD2_THREADS), FWD2_SMEM_BYTES, stream, tq, tk, tv, p, 1));
    dim3 gc((a->s + 3) / 4, a->hq, a->b);
    B200TP_CUDA_OK(launch_pdl(flash_fwd_combine_kernel, gc, dim3(128), 0, stream, a->s, a->hq, D, ns, p.split_min,
                              a->seg_start, static_cast<const float*>(p.o_part), static_cast<const float*>(p.ml_part),
                              p.out, p.out_sb, p.out_sh, p.out_ss, lse));
    return B200TP_OK;
  }
  const int fwd_choice = a->reserved & 3;
  if (fwd_choice == 1 || (fwd_choice != 2 && two_tile_ctas <= sm_count())) {
    // single-tile kernel (reserved & 3 == 1 / 2 force the single- / two-tile kernel, for cross-checks)
    dim3 grid(a->hq * a->b, nqb, 1);
    B200TP_CUDA_OK(launch_pdl(flash_fwd_kernel<D>, grid, dim3(FWD_THREADS), FWD_SMEM_BYTES, stream, tq, tk, tv, p));
  } else if (group % 2 == 0) {
    dim3 grid(a->hq / 2 * a->b, nqb, 1);       // two heads of a GQA group per CTA
    B200TP_CUDA_OK(launch_pdl(flash_fwd2_kernel<D>, grid, dim3(FWD2_THREADS), FWD2_SMEM_BYTES, stream, tq, tk, tv, p, 1));
  } else {
    dim3 grid(a->hq * a->b, (nqb + 1) / 2, 1); // two consecutive query blocks of a head per CTA
    B200TP_CUDA_OK(launch_pdl(flash_fwd2_kernel<D>, grid, dim3(FWD2_THREADS), FWD2_SMEM_BYTES, stream, tq, tk, tv, p, 0));
  }
  return B200TP_OK;
}

int flash_tc_fwd(const b200tp_attn_args* a, const void* q, const void* k, const void* v, void* o, float* lse,
                 void* workspace, size_t workspace_bytes, cudaStream_t stream, int* status) {
  switch (a->d) {
    case 64: return fwd_impl<64>(a, q, k, v, o, lse, workspace, workspace_bytes, stream, status);
    case 96: return fwd_impl<96>(a, q, k, v, o, lse, workspace, workspace_bytes, stream, status);
    case 128: return fwd_impl<128>(a, q, k, v, o, lse, workspace, workspace_bytes, stream, status);
    default: return fail(B200TP_ERR_UNSUPPORTED_ATTN, "head_dim must be 64, 96 or 128");
  }
}

#ifdef B200TP_TRACE
extern "C" int b200tp_debug_trace(long long* host, int count) {
  return static_cast<int>(cudaMemcpyFromSymbol(host, g_trace, sizeof(long long) * count));
}
#endif

// q heads one dK / dV CTA covers: the whole GQA group when the grid of (kv head, key block) CTAs still
// holds about 1.7 per SM (heaviest-first dispatch then balances them), one otherwise (more, smaller CTAs
// and fp32 per-q-head partials).  reserved & 64 forces one, reserved & 128 the group (cross-checks).
static int dkv_heads_per_cta(const b200tp_attn_args* a) {
  const int group = a->hq / a->hkv;
  if (group == 1 || (a->reserved & 64)) return 1;
  if (a->reserved & 128) return group;
  const long long ctas = static_cast<long long>(a->b) * a->hkv * ((a->s + TILE - 1) / TILE);
  return 10 * ctas >= 17LL * sm_count() ? group : 1;   // measured: wins from 256 CTAs on 148 SMs, loses at 128
}

// The statistics tile the dQ kernel leaves for the dK / dV kernel (32 bytes per query row, whole 64-row
// blocks), and the fp32 per-q-head dK / dV partials when query heads share kv heads and each has its own CTAs.
static int stat_blocks_per_head(const b200tp_attn_args* a) { return 2 * ((a->s + TILE - 1) / TILE); }
static size_t stat_bytes(const b200tp_attn_args* a) {
  return align_up(static_cast<size_t>(a->b) * a->hq * stat_blocks_per_head(a) * 2048, 256);
}
size_t flash_tc_bwd_workspace_bytes(const b200tp_attn_args* a) {
  if (a->hq == a->hkv || dkv_heads_per_cta(a) > 1) return stat_bytes(a);
  return stat_bytes(a) + 2 * align_up(static_cast<size_t>(a->b) * a->hq * a->s * HD * sizeof(float), 256);
}

template <int D>
static int bwd_impl(const b200tp_attn_args* a, const void* q, const void* k, const void* v, const void* o,
                    const float* lse, const void* d_o, void* dq, void* dk, void* dv, void* workspace,
                    cudaStream_t stream, int* status) {
  int rc = configure();
  if (rc) return rc;
  if (!(a->scale > 0.f)) return fail(B200TP_ERR_ATTN_INPUT, "scale must be positive");
  const size_t part_bytes = align_up(static_cast<size_t>(a->b) * a->hq * a->s * HD * sizeof(float), 256);
  float* dk_part = nullptr;
  float* dv_part = nullptr;
  __nv_bfloat16* stat = static_cast<__nv_bfloat16*>(workspace);
  const int stat_blocks = stat_blocks_per_head(a);
  const size_t after_stat = stat_bytes(a);
  const int dkv_heads = dkv_heads_per_cta(a);
  if (a->hq != a->hkv && dkv_heads == 1) {
    dk_part = reinterpret_cast<float*>(static_cast<char*>(workspace) + after_stat);
    dv_part = reinterpret_cast<float*>(static_cast<char*>(workspace) + after_stat + part_bytes);
  }
  CUtensorMap tq, tk, tv, tdo;
  rc = make_tmap_bhsd_bf16(&tq, q, a->b, a->hq, a->s, D, a->q_stride[0], a->q_stride[1], a->q_stride[2], TILE, 64);
  if (rc) return rc;
  rc = make_tmap_bhsd_bf16(&tk, k, a->b, a->hkv, a->s, D, a->k_stride[0], a->k_stride[1], a->k_stride[2], TILE, 64);
  if (rc) return rc;
  rc = make_tmap_bhsd_bf16(&tv, v, a->b, a->hkv, a->s, D, a->v_stride[0], a->v_stride[1], a->v_stride[2], TILE, 64);
  if (rc) return rc;
  rc = make_tmap_bhsd_bf16(&tdo, d_o, a->b, a->hq, a->s, D, a->o_stride[0], a->o_stride[1], a->o_stride[2], TILE, 64);
  if (rc) return rc;
  CUtensorMap tq64, tk64, tv64, tdo64;  // 64-row boxes for the operand that is streamed in half tiles
  rc = make_tmap_bhsd_bf16(&tq64, q, a->b, a->hq, a->s, D, a->q_stride[0], a->q_stride[1], a->q_stride[2], 64, 64);
  if (rc) return rc;
  rc = make_tmap_bhsd_bf16(&tk64, k, a->b, a->hkv, a->s, D, a->k_stride[0], a->k_stride[1], a->k_stride[2], 64, 64);
  if (rc) return rc;
  rc = make_tmap_bhsd_bf16(&tv64, v, a->b, a->hkv, a->s, D, a->v_stride[0], a->v_stride[1], a->v_stride[2], 64, 64);
  if (rc) return rc;
  rc = make_tmap_bhsd_bf16(&tdo64, d_o, a->b, a->hq, a->s, D, a->o_stride[0], a->o_stride[1], a->o_stride[2], 64, 64);
  if (rc) return rc;

  // Row statistics (-D, -L log2 e): formed by the dQ kernel for its own rows and published for the dK / dV
  // kernel; the stand-alone pre-pass only runs when the dQ kernel is left out (timing of dK / dV alone).
  if (a->reserved & 512) {
    dim3 gd(stat_blocks * 16, a->hq, a->b);   // four rows per block, whole 64-row blocks of the statistics tile
    B200TP_CUDA_OK(launch_pdl(bwd_d_kernel, gd, dim3(128), 0, stream, a->s, a->hq, D,
                              static_cast<const __nv_bfloat16*>(d_o), static_cast<const __nv_bfloat16*>(o),
                              static_cast<long long>(a->o_stride[0]), static_cast<long long>(a->o_stride[1]),
                              static_cast<long long>(a->o_stride[2]), lse, stat, stat_blocks,
                              a->scale * kLog2e));
  }

  AttnParams p = base_params(a, status);
  p.lse = lse;
  p.o_saved = static_cast<const __nv_bfloat16*>(o);
  p.stat_w = stat;
  p.stat = stat;
  p.stat_blocks = stat_blocks;
  p.out = static_cast<__nv_bfloat16*>(dq);
  p.out_sb = a->q_stride[0]; p.out_sh = a->q_stride[1]; p.out_ss = a->q_stride[2];
  p.dk = static_cast<__nv_bfloat16*>(dk);
  p.dv = static_cast<__nv_bfloat16*>(dv);
  p.dk_sb = a->k_stride[0]; p.dk_sh = a->k_stride[1]; p.dk_ss = a->k_stride[2];
  p.dv_sb = a->v_stride[0]; p.dv_sh = a->v_stride[1]; p.dv_ss = a->v_stride[2];
  const int nqb = (a->s + TILE - 1) / TILE;
  // reserved & 512 / & 256 leave out the dQ / the dK, dV kernel: lets a benchmark time each alone
  if (!(a->reserved & 512)) {
    dim3 gq(a->hq * a->b, nqb, 1);
    B200TP_CUDA_OK(launch_pdl(flash_dq_kernel<D>, gq, dim3(DQ_THREADS), DQ_SMEM_BYTES, stream, tk64, tv64,
                              static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(d_o),
                              static_cast<long long>(a->q_stride[0]), static_cast<long long>(a->q_stride[1]),
                              static_cast<long long>(a->q_stride[2]), static_cast<long long>(a->o_stride[0]),
                              static_cast<long long>(a->o_stride[1]), static_cast<long long>(a->o_stride[2]), p));
  }
  if (a->reserved & 256) return B200TP_OK;
  p.dk_part = dk_part;
  p.dv_part = dv_part;
  p.dkv_heads = dkv_heads;
  dim3 gk(a->hq / dkv_heads * a->b, nqb, 1);
  B200TP_CUDA_OK(launch_pdl(flash_dkv_kernel<D>, gk, dim3(DKV_THREADS), DKV_SMEM_BYTES, stream, tq64, tk, tv, tdo64, p));
  if (dk_part != nullptr) {
    const long long total = static_cast<long long>(a->b) * a->hkv * a->s * (D / 8);
    B200TP_CUDA_OK(launch_pdl(dkv_reduce_kernel, dim3(static_cast<unsigned>((total + 255) / 256)), dim3(256), 0, stream,
                              a->b, a->hq, a->hkv, a->s, D, a->scale, static_cast<const float*>(dk_part),
                              static_cast<const float*>(dv_part), static_cast<__nv_bfloat16*>(dk),
                              static_cast<__nv_bfloat16*>(dv), static_cast<long long>(a->k_stride[0]),
                              static_cast<long long>(a->k_stride[1]), static_cast<long long>(a->k_stride[2]),
                              static_cast<long long>(a->v_stride[0]), static_cast<long long>(a->v_stride[1]),
                              static_cast<long long>(a->v_stride[2])));
  }
  return B200TP_OK;
}

int flash_tc_bwd(const b200tp_attn_args* a, const void* q, const void* k, const void* v, const void* o,
                 const float* lse, const void* d_o, void* dq, void* dk, void* dv, void* workspace, cudaStream_t stream,
                 int* status) {
  switch (a->d) {
    case 64: return bwd_impl<64>(a, q, k, v, o, lse, d_o, dq, dk, dv, workspace, stream, status);
    case 96: return bwd_impl<96>(a, q, k, v, o, lse, d_o, dq, dk, dv, workspace, stream, status);
    case 128: return bwd_impl<128>(a, q, k, v, o, lse, d_o, dq, dk, dv, workspace, stream, status);
    default: return fail(B200TP_ERR_UNSUPPORTED_ATTN, "head_dim must be 64, 96 or 128");
  }
}

}  // namespace b200tp
