// Fused linear cross-entropy on the Blackwell tensor cores (tcgen05 / TMEM / TMA).
//
// Four kernels:
//
//  ce_logits_kernel<FWD>    Z = H W^T tile by tile (128 rows x 256 vocab columns, K = D),
//                           accumulators double-buffered in tensor memory; the epilogue
//                           warps fold each tile into a per-row online (max, sum-exp,
//                           target-logit) and write ONE partial triple per (row, vocab
//                           split).  The logits never leave the SM.
//  ce_logits_kernel<BWD_G>  same main loop over one vocab chunk; the epilogue forms
//                           g = (exp(z - lse) - onehot) * cotangent, rounds it to bf16 and
//                           stores it to a (N, chunk) scratch matrix.
//  ce_dh_kernel             dH(128 x 256 tile) (+)= G(N, chunk) W[chunk, :] with the vocab
//                           axis as the contraction: A = G is K-major, B = W is read as an
//                           MN-major operand straight from its row-major storage.
//  ce_dw_kernel             trainable heads: dW_chunk(128 x 256 tile) = G^T hidden with the token
//                           axis as the contraction; both operands read MN-major from their
//                           row-major storage, written once (each vocab row has one chunk).
//
// Work split: persistent CTAs (one per SM), static round-robin over work units.  Roles in
// a CTA of 192 threads: warp 0 = TMA producer, warp 1 = MMA issuer (also owns the TMEM
// allocation), warps 2..5 = epilogue (one TMEM lane quadrant each).
//
// 4-bit affine group-64 heads (QUANT instantiations of ce_logits_kernel and ce_dh_kernel): the
// weight operand is never materialised in global memory.  The TMA producer copies the packed codes
// of each stage's weight tile into a small shared-memory ring (8 KiB per stage) beside the other
// operand; eight more warps (256 threads, one (vocab row, 64-column group) each per stage) read
// their 32 bytes of codes from there and the group's scale / bias from global memory (prefetched in
// registers), expand them (dequant.cuh) and write the bf16 tile into the stage's swizzled slot,
// where the MMA reads it exactly as it reads a TMA-loaded dense tile.
// core/kernel/source.py:199-340 (K2) and core/kernel/launch.py:336-373.
//
// Replaces core/kernel/source.py:25-166 (forward MSL), :475-611 (dH MMA backward), :659-702 (dW)
// and the chunked backward of core/chunked.py:52-90 of the reference.
#include "linear_ce_tc.h"

#include <algorithm>
#include <atomic>
#include <map>
#include <mutex>
#include <tuple>
#include <vector>

#include "dequant.cuh"
#include "ptx.cuh"

namespace b200tp {

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;  // 16 KiB
constexpr int B_BYTES = BN * BK * 2;  // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int THREADS = 192;
constexpr int DQ_WARPS = 8;                       // dequantising warps of the QUANT kernels
constexpr int THREADS_Q = THREADS + 32 * DQ_WARPS;
constexpr int DQ_FULL_ARRIVALS = DQ_WARPS;        // one arrival per dequantising warp on a stage's full barrier
constexpr int CODE_BYTES = 32 * 1024;             // QUANT: ring of packed-code tiles filled by TMA
constexpr int CODE_SLOTS_LOGITS = 2;              // 256 rows x 64 B (two k blocks) = 16 KiB each
constexpr int CODE_SLOTS_DH = 4;                  // 64 rows x 128 B (one k block, 256 columns) = 8 KiB each
constexpr int BAR_BYTES = 256;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + 1024;  // + alignment slack
constexpr int SMEM_BYTES_Q = SMEM_BYTES + CODE_BYTES;
constexpr uint32_t TMEM_COLS = 512;                                  // two 256-column accumulators

enum { MODE_FWD = 0, MODE_BWD_G = 1 };


struct LogitsParams {
  int n_rows;            // N
  int k_dim;             // D
  int vrow0, vrow1;      // rows of the weight matrix (tensor map coordinates) this launch covers
  long long vocab_id0;   // global vocab id of tensor-map row 0
  int num_rb, num_vt, splits;
  const long long* targets;
  long long ignore_index;
  // FWD: partial triples, [split][N] each
  float* pm;
  float* ps;
  float* pt;
  // BWD_G
  const float* lse;
  const float* ct;
  __nv_bfloat16* g;
  int ldg;
  int* status;
  // QUANT: the packed head (rows indexed like the tensor map of a dense weight would be)
  const uint32_t* wq;
  const void* scales;
  const void* biases;
  int qp_f32;
  int qvec;              // bf16 scales / biases, D % 512 == 0, 16-byte aligned: eight groups per load
};

struct DhParams {
  int n_rows;     // N
  int d_cols;     // D
  int k_total;    // contraction length (multiple of 64; columns of G)
  int wrow0;      // first vocab row of this chunk in the weight tensor map
  int num_rb, num_nt;
  const float* acc_in;   // fp32 (N, D) partial sums to add, or nullptr
  float* acc_out;        // fp32 (N, D) destination, or nullptr
  __nv_bfloat16* out_bf16;  // bf16 (N, D) destination, or nullptr
  int* status;
  int tile0, tile1;         // tiles [tile0, tile1) of the row-block-major order are computed by this launch
  // QUANT: the packed head
  const uint32_t* wq;
  const void* scales;
  const void* biases;
  int qp_f32;
  int w_rows;               // vocab rows of the head (rows at or past it read as zero)
};

struct DwParams {
  int n_rows;     // N tokens = contraction length
  int d_cols;     // D
  int v_rows;     // vocab rows of this chunk (rows of the d_weight block written)
  int num_mt, num_nt;
  __nv_bfloat16* out;   // (v_rows, D) bf16 block of d_weight, row stride D
  int* status;
};

struct SmemView {
  uint8_t* base;
  uint64_t* full;
  uint64_t* empty;
  uint64_t* tfull;
  uint64_t* tempty;
  uint32_t* tmem_ptr;
  int* abort_flag;
  uint8_t* codes;       // QUANT only
  uint64_t* cfull;      // [4]
  uint64_t* cempty;     // [4]
  __device__ uint8_t* a(int s) const { return base + s * STAGE_BYTES; }
  __device__ uint8_t* b(int s) const { return base + s * STAGE_BYTES + A_BYTES; }
};

__device__ __forceinline__ SmemView carve_smem(uint8_t* raw, bool quant = false) {
  const uint32_t addr = smem_u32(raw);
  const uint32_t aligned = (addr + 1023u) & ~1023u;
  SmemView v;
  v.base = raw + (aligned - addr);
  v.codes = v.base + STAGES * STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(v.base + STAGES * STAGE_BYTES + (quant ? CODE_BYTES : 0));
  v.cfull = bars + 2 * STAGES + 6;
  v.cempty = bars + 2 * STAGES + 10;
  v.full = bars;
  v.empty = bars + STAGES;
  v.tfull = bars + 2 * STAGES;
  v.tempty = bars + 2 * STAGES + 2;
  v.tmem_ptr = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  v.abort_flag = reinterpret_cast<int*>(v.tmem_ptr + 1);
  return v;
}

// A dequantising warp's part of "the stage's weight tile is written": every thread fences its own
// generic-proxy stores against the tensor core's async proxy, then one lane arrives for the warp.
__device__ __forceinline__ void dq_signal_written(uint64_t* full_bar, int lane) {
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0) mbar_arrive(full_bar);
}

__device__ __forceinline__ void raise_abort(const SmemView& sm, int* status, int code) {
  atomicExch(sm.abort_flag, 1);
  if (status != nullptr) atomicCAS(status, 0, code);
}

// Common prologue: barriers, TMEM allocation.  Returns the TMEM base address.
__device__ __forceinline__ uint32_t cta_setup(const SmemView& sm, int warp, uint32_t full_count = 1) {
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sm.full[s], full_count);   // the TMA producer's arrive.expect_tx (+ one per dequantising warp)
      mbar_init(&sm.empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sm.tfull[s], 1);
      mbar_init(&sm.tempty[s], 4);  // one arrive per epilogue warp
    }
    if (full_count > 1) {
      for (int s = 0; s < 4; ++s) {
        mbar_init(&sm.cfull[s], 1);
        mbar_init(&sm.cempty[s], DQ_WARPS);
      }
    }
    *sm.abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(sm.tmem_ptr, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  return *reinterpret_cast<volatile uint32_t*>(sm.tmem_ptr);
}

__device__ __forceinline__ void cta_teardown(const SmemView& sm, int warp, uint32_t tmem_base) {
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// After an abort the producer may still have bulk copies in flight into this CTA's shared
// memory: wait (bounded) for every stage it armed before the CTA is allowed to retire.
__device__ __forceinline__ void producer_drain(const SmemView& sm, uint32_t it) {
  const uint32_t first = it > STAGES ? it - STAGES : 0;
  for (uint32_t j = first; j < it; ++j) mbar_wait_drain(&sm.full[j % STAGES], (j / STAGES) & 1);
}

// -----------------------------------------------------------------------------------------
// Z = H W^T with fused epilogues
// -----------------------------------------------------------------------------------------
// Walk over the (work unit, vocab tile, k block) sequence of one persistent CTA, in the order the
// producer, the MMA issuer and the dequantising warps all follow.
struct LogitsWalk {
  int u, vt, vt1, kb;
  __device__ __forceinline__ void set_unit(const LogitsParams& p) {
    const int split = u / p.num_rb;
    vt = static_cast<int>(static_cast<long long>(split) * p.num_vt / p.splits);
    vt1 = static_cast<int>(static_cast<long long>(split + 1) * p.num_vt / p.splits);
    kb = 0;
  }
  __device__ __forceinline__ void init(const LogitsParams& p, int total_units) {
    u = blockIdx.x;
    if (u < total_units) set_unit(p);
  }
  __device__ __forceinline__ void next(const LogitsParams& p, int total_units, int kblocks) {
    if (++kb < kblocks) return;
    kb = 0;
    if (++vt < vt1) return;
    u += gridDim.x;
    if (u < total_units) set_unit(p);
  }
};

template <int MODE, bool QUANT>
__global__ void __launch_bounds__(QUANT ? THREADS_Q : THREADS, 1)
ce_logits_kernel(const __grid_constant__ CUtensorMap tmap_h, const __grid_constant__ CUtensorMap tmap_w,
                 const LogitsParams p) {
  extern __shared__ uint8_t smem_raw[];
  const SmemView sm = carve_smem(smem_raw, QUANT);
  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);   // provably warp-uniform
  const int lane = threadIdx.x & 31;
  const uint32_t tmem_base = cta_setup(sm, warp, QUANT ? 1 + DQ_FULL_ARRIVALS : 1);

  const int total_units = p.num_rb * p.splits;
  const int kblocks = (p.k_dim + BK - 1) / BK;

  if (QUANT && warp >= THREADS / 32) {
    // ------------------------------ dequantising warps ------------------------------
    // Thread t owns row t of the stage's 256-row weight tile: one group of 64 codes per k block.  A code
    // tile (256 rows x 64 bytes, 64-byte swizzle) holds two k blocks.  Scales / biases: eight groups per
    // 16-byte load, one load ahead (`qvec`: bf16 parameters, D % 512 == 0), else one load per stage.
    const int trow = threadIdx.x - THREADS;
    const int groups = p.k_dim / 64;
    const bool qp_f32 = p.qp_f32 != 0, qvec = p.qvec != 0;
    const uint32_t swz = static_cast<uint32_t>((trow >> 1) & 3);
    LogitsWalk cur;
    cur.init(p, total_units);
    auto row_of = [&](const LogitsWalk& w) { return p.vrow0 + w.vt * BN + trow; };
    auto load8 = [&](const LogitsWalk& w, uint4& s8, uint4& b8) {
      const int row = row_of(w);
      if (row < p.vrow1) {
        const long long idx = static_cast<long long>(row) * groups + (w.kb & ~7);
        s8 = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned short*>(p.scales) + idx));
        b8 = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned short*>(p.biases) + idx));
      }
    };
    auto pick = [](const uint4& v, int k) -> uint32_t {   // k-th bf16 of eight
      const uint32_t lo = (k & 4) ? v.z : v.x, hi = (k & 4) ? v.w : v.y;
      return (((k & 2) ? hi : lo) >> ((k & 1) * 16)) & 0xFFFFu;
    };
    uint4 s_cur = make_uint4(0, 0, 0, 0), b_cur = s_cur, s_nxt = s_cur, b_nxt = s_cur;
    LogitsWalk pre = cur;      // start of the eight-block span after the current one
    if (qvec && cur.u < total_units) {
      load8(cur, s_nxt, b_nxt);
    }
    uint32_t it = 0, ci = 0;
    bool ok = true;
#pragma unroll 1
    for (; cur.u < total_units && ok; cur.next(p, total_units, kblocks), ++it) {
      const int row = row_of(cur);
      const bool valid = row < p.vrow1;
      uint32_t sc, bi;
      if (qvec) {
        if ((cur.kb & 7) == 0) {
          s_cur = s_nxt;
          b_cur = b_nxt;
          // the span after this one: eight k blocks on, or the next tile / unit (kblocks % 8 == 0 here)
          pre = cur;
          for (int k = 0; k < 8 && pre.u < total_units; ++k) pre.next(p, total_units, kblocks);
          if (pre.u < total_units) load8(pre, s_nxt, b_nxt);
        }
        sc = pick(s_cur, cur.kb & 7);
        bi = pick(b_cur, cur.kb & 7);
      } else {
        sc = bi = 0;
        if (valid) {
          sc = dq_load_param(p.scales, static_cast<long long>(row) * groups + cur.kb, qp_f32);
          bi = dq_load_param(p.biases, static_cast<long long>(row) * groups + cur.kb, qp_f32);
        }
      }
      // ---- this row's 32 bytes of codes from the TMA-filled tile (two k blocks per tile)
      const int half = cur.kb & 1;
      const uint32_t cs = ci % CODE_SLOTS_LOGITS;
      if (half == 0 && !mbar_wait_warp(&sm.cfull[cs], (ci / CODE_SLOTS_LOGITS) & 1, sm.abort_flag)) {
        if (lane == 0) raise_abort(sm, p.status, kDevTimeoutProducer);
        ok = false;
        break;
      }
      const uint32_t crow = smem_u32(sm.codes) + cs * (CODE_BYTES / CODE_SLOTS_LOGITS) + trow * 64;
      const uint4 lo = lds128(crow + (((2 * half) ^ swz) << 4));
      const uint4 hi = lds128(crow + (((2 * half + 1) ^ swz) << 4));
      const bool release_codes = half == 1 || cur.kb + 1 == kblocks;   // last k block served by this tile
      const int s = it % STAGES;
      if (!mbar_wait_warp(&sm.empty[s], ((it / STAGES) & 1) ^ 1, sm.abort_flag)) {
        if (lane == 0) raise_abort(sm, p.status, kDevTimeoutProducer);
        ok = false;
        break;
      }
      dq_store_row(smem_u32(sm.b(s)) + trow * 128, trow & 7, lo, hi, sc, bi, qp_f32, valid);
      dq_signal_written(&sm.full[s], lane);
      // The code slot goes back to the producer only now, after `lo` / `hi` have been consumed: an
      // mbarrier arrive issued right behind the shared-memory loads can be performed before those loads
      // have read their data when the load / store unit is backed up (observed: with the backward's
      // epilogue streaming G to global memory, the producer's refill overwrote rows a warp had not read yet).
      if (release_codes) {
        if (lane == 0) mbar_arrive(&sm.cempty[cs]);
        ++ci;
      }
    }
  } else if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmap_h);
      tma_prefetch_desc(&tmap_w);
      uint32_t it = 0, ci = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
        const int split = u / p.num_rb;
        const int rb = u - split * p.num_rb;
        const int vt0 = static_cast<int>(static_cast<long long>(split) * p.num_vt / p.splits);
        const int vt1 = static_cast<int>(static_cast<long long>(split + 1) * p.num_vt / p.splits);
        for (int vt = vt0; vt < vt1 && ok; ++vt) {
          for (int kb = 0; kb < kblocks; ++kb, ++it) {
            const int s = it % STAGES;
            if (!mbar_wait(&sm.empty[s], ((it / STAGES) & 1) ^ 1, sm.abort_flag)) {
              raise_abort(sm, p.status, kDevTimeoutProducer);
              ok = false;
              break;
            }
            if (QUANT && (kb & 1) == 0) {
              // packed codes of k blocks kb, kb + 1 for the tile's 256 rows (tmap_w is the uint32 map here)
              const uint32_t cs = ci % CODE_SLOTS_LOGITS;
              if (!mbar_wait(&sm.cempty[cs], ((ci / CODE_SLOTS_LOGITS) & 1) ^ 1, sm.abort_flag)) {
                raise_abort(sm, p.status, kDevTimeoutProducer);
                ok = false;
                break;
              }
              mbar_arrive_expect_tx(&sm.cfull[cs], CODE_BYTES / CODE_SLOTS_LOGITS);
              tma_load_2d(sm.codes + cs * (CODE_BYTES / CODE_SLOTS_LOGITS), &tmap_w, &sm.cfull[cs], kb * 8,
                          p.vrow0 + vt * BN);
              ++ci;
            }
            mbar_arrive_expect_tx(&sm.full[s], QUANT ? A_BYTES : STAGE_BYTES);
            tma_load_2d(sm.a(s), &tmap_h, &sm.full[s], kb * BK, rb * BM);
            if (!QUANT) tma_load_2d(sm.b(s), &tmap_w, &sm.full[s], kb * BK, p.vrow0 + vt * BN);
          }
        }
      }
      if (!ok) {
        producer_drain(sm, it);
        if (QUANT)
          for (uint32_t c = ci > CODE_SLOTS_LOGITS ? ci - CODE_SLOTS_LOGITS : 0; c < ci; ++c)
            mbar_wait_drain(&sm.cfull[c % CODE_SLOTS_LOGITS], (c / CODE_SLOTS_LOGITS) & 1);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    // The whole warp runs the loop (its address arithmetic stays warp-uniform and cheap: this warp
    // shares an instruction scheduler with epilogue warps) and one elected lane issues.
    constexpr uint32_t idesc = make_idesc_bf16(BM, BN, 0, 0);
    constexpr uint32_t dhi = desc_hi_sw128(1024);
    uint32_t it = 0, tile = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
      const int split = u / p.num_rb;
      const int vt0 = static_cast<int>(static_cast<long long>(split) * p.num_vt / p.splits);
      const int vt1 = static_cast<int>(static_cast<long long>(split + 1) * p.num_vt / p.splits);
      for (int vt = vt0; vt < vt1 && ok; ++vt, ++tile) {
        const uint32_t as = tile & 1;
        if (!mbar_wait_warp(&sm.tempty[as], ((tile >> 1) & 1) ^ 1, sm.abort_flag)) {
          if (lane == 0) raise_abort(sm, p.status, kDevTimeoutMma);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + as * BN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait_warp(&sm.full[s], (it / STAGES) & 1, sm.abort_flag)) {
            if (lane == 0) raise_abort(sm, p.status, kDevTimeoutMma);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_lo = desc_lo(smem_u32(sm.a(s)), 16);
          const uint32_t b_lo = desc_lo(smem_u32(sm.b(s)), 16);
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < BK / 16; ++k)
              umma_ss_w(d_tmem, a_lo + k * 2, dhi, b_lo + k * 2, dhi, idesc, (kb | k) != 0 ? 1u : 0u);
            umma_commit(&sm.empty[s]);  // frees the stage once these MMAs have read it
          }
          __syncwarp();
        }
        if (ok && elect_one()) umma_commit(&sm.tfull[as]);
        __syncwarp();
      }
    }
  } else {
    // ------------------------------ epilogue warps ------------------------------
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    const int row_in_tile = quad * 32 + lane;
    uint32_t tile = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
      const int split = u / p.num_rb;
      const int rb = u - split * p.num_rb;
      const int vt0 = static_cast<int>(static_cast<long long>(split) * p.num_vt / p.splits);
      const int vt1 = static_cast<int>(static_cast<long long>(split + 1) * p.num_vt / p.splits);
      const int row = rb * BM + row_in_tile;
      const bool row_ok = row < p.n_rows;
      long long target = p.ignore_index;
      if (row_ok) target = p.targets[row];
      const bool tvalid = row_ok && target != p.ignore_index;

      float run_m = -INFINITY, run_s = 0.f, run_t = 0.f;  // FWD state (log2 domain for m)
      float lse2 = 0.f, ctv = 0.f;                        // BWD_G state
      if (MODE == MODE_BWD_G && row_ok) {
        lse2 = p.lse[row] * kLog2e;
        ctv = tvalid ? p.ct[row] : 0.f;
      }

      for (int vt = vt0; vt < vt1 && ok; ++vt, ++tile) {
        const uint32_t as = tile & 1;
        if (!mbar_wait_warp(&sm.tfull[as], (tile >> 1) & 1, sm.abort_flag)) {
          raise_abort(sm, p.status, kDevTimeoutEpilogue);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const int tile_row0 = p.vrow0 + vt * BN;                      // tensor-map row of column 0
        const int ncols = min(BN, p.vrow1 - tile_row0);               // valid columns in this tile
        long long trel = -1;
        if (tvalid) trel = target - (p.vocab_id0 + tile_row0);
        const int tcol = (trel >= 0 && trel < ncols) ? static_cast<int>(trel) : -1;
        const uint32_t taddr0 = tmem_base + as * BN + (static_cast<uint32_t>(quad * 32) << 16);

#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          if (MODE == MODE_FWD && c * 32 >= ncols) break;
          uint32_t r[32];
          tmem_ld_x32(taddr0 + c * 32, r);
          tmem_wait_ld();
          tmem_regs_ready(r);
          const int cvalid = ncols - c * 32;  // columns of this chunk that exist (may exceed 32)
          if (MODE == MODE_FWD) {
            float x[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              x[j] = __uint_as_float(r[j]);
              if (j >= cvalid) x[j] = -INFINITY;
            }
            if (tcol >= 0 && (tcol >> 5) == c) {
              const int tj = tcol & 31;
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (j == tj) run_t = x[j];
            }
            float cm = x[0];
#pragma unroll
            for (int j = 1; j < 32; ++j) cm = fmaxf(cm, x[j]);
            // cm is finite: column c*32 exists (checked above) and logits are finite.
            const float new_m = fmaxf(run_m, cm * kLog2e);
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < 32; ++j) acc += fast_exp2(fmaf(x[j], kLog2e, -new_m));
            run_s = run_s * fast_exp2(run_m - new_m) + acc;
            run_m = new_m;
          } else {
            uint32_t packed[16];
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              float g0 = fast_exp2(fmaf(__uint_as_float(r[j]), kLog2e, -lse2));
              float g1 = fast_exp2(fmaf(__uint_as_float(r[j + 1]), kLog2e, -lse2));
              if (c * 32 + j == tcol) g0 -= 1.f;
              if (c * 32 + j + 1 == tcol) g1 -= 1.f;
              g0 = (j < cvalid) ? g0 * ctv : 0.f;
              g1 = (j + 1 < cvalid) ? g1 * ctv : 0.f;
              packed[j >> 1] = pack_bf16x2(g0, g1);
            }
            if (row_ok) {
              uint4* dst = reinterpret_cast<uint4*>(p.g + static_cast<size_t>(row) * p.ldg + vt * BN + c * 32);
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4)
                dst[q4] = make_uint4(packed[4 * q4], packed[4 * q4 + 1], packed[4 * q4 + 2], packed[4 * q4 + 3]);
            }
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.tempty[as]);
      }

      if (MODE == MODE_FWD && ok && row_ok) {
        const size_t o = static_cast<size_t>(split) * p.n_rows + row;
        p.pm[o] = run_m * kLn2;  // back to natural-log units
        p.ps[o] = run_s;
        p.pt[o] = run_t;
      }
    }
  }
  cta_teardown(sm, warp, tmem_base);
}

// -----------------------------------------------------------------------------------------
// dH (+)= G W_chunk
// -----------------------------------------------------------------------------------------
// Tiles are numbered row-block-major (t = rb * num_nt + nt), so the row blocks of d_hidden complete
// in order as the persistent CTAs advance, and a launch can be given a sub-range [tile0, tile1) of
// them: vocab-sharded callers run the last chunk in a few such launches and start reducing the
// finished rows across ranks while the later ones are still being computed.
template <bool QUANT>
__global__ void __launch_bounds__(QUANT ? THREADS_Q : THREADS, 1)
ce_dh_kernel(const __grid_constant__ CUtensorMap tmap_g, const __grid_constant__ CUtensorMap tmap_w,
             const DhParams p) {
  extern __shared__ uint8_t smem_raw[];
  const SmemView sm = carve_smem(smem_raw, QUANT);
  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);   // provably warp-uniform
  const int lane = threadIdx.x & 31;
  const uint32_t tmem_base = cta_setup(sm, warp, QUANT ? 1 + DQ_FULL_ARRIVALS : 1);

  const int total_tiles = p.tile1;
  const int first_tile = p.tile0 + blockIdx.x;
  const int kblocks = p.k_total / BK;

  if (QUANT && warp >= THREADS / 32) {
    // ------------------------------ dequantising warps ------------------------------
    // Stage tile: 64 vocab rows (k) x 256 hidden columns as four [64 k][64 n] boxes = four groups per
    // vocab row.  Warp w, lane l: vocab row 8 w + (l & 7), box l >> 3 -- eight consecutive rows per
    // quarter-warp, so the reads of the code tile (64 rows x 128 B, 128-byte swizzle), the writes of the
    // operand tile and the scale / bias loads (four consecutive values per row) are all conflict-free /
    // coalesced.  Scales and biases are prefetched three stages ahead in registers.
    const int dw = warp - THREADS / 32;
    const int krow = dw * 8 + (lane & 7), box = lane >> 3;
    const int groups = p.d_cols / 64;
    const bool qp_f32 = p.qp_f32 != 0;
    constexpr int PF = 3;
    int t_cur = first_tile, kb_cur = 0, t_pre = first_tile, kb_pre = 0;
    uint32_t sc_ring[PF], bi_ring[PF];
    auto coords = [&](int t, int kb, int& row, int& col) {
      const int nt = t % p.num_nt;
      row = p.wrow0 + kb * BK + krow;
      col = nt * BN + box * 64;
    };
    auto fetch = [&](uint32_t& sc, uint32_t& bi, int t, int kb) {
      int row, col;
      coords(t, kb, row, col);
      sc = bi = 0;
      if (row < p.w_rows && col < p.d_cols) {
        const long long idx = static_cast<long long>(row) * groups + col / 64;
        sc = dq_load_param(p.scales, idx, qp_f32);
        bi = dq_load_param(p.biases, idx, qp_f32);
      }
    };
    auto advance = [&](int& t, int& kb) {
      if (++kb == kblocks) {
        kb = 0;
        t += gridDim.x;
      }
    };
#pragma unroll
    for (int j = 0; j < PF; ++j) {
      if (t_pre < total_tiles) {
        fetch(sc_ring[j], bi_ring[j], t_pre, kb_pre);
        advance(t_pre, kb_pre);
      }
    }
    uint32_t it = 0;
    bool ok = true;
#pragma unroll 1
    while (t_cur < total_tiles && ok) {
#pragma unroll
      for (int j = 0; j < PF; ++j) {
        if (t_cur >= total_tiles || !ok) break;
        const uint32_t sc = sc_ring[j], bi = bi_ring[j];
        int row, col;
        coords(t_cur, kb_cur, row, col);
        const bool valid = row < p.w_rows && col < p.d_cols;
        if (t_pre < total_tiles) {
          fetch(sc_ring[j], bi_ring[j], t_pre, kb_pre);
          advance(t_pre, kb_pre);
        }
        const uint32_t cs = it % CODE_SLOTS_DH;
        if (!mbar_wait_warp(&sm.cfull[cs], (it / CODE_SLOTS_DH) & 1, sm.abort_flag)) {
          if (lane == 0) raise_abort(sm, p.status, kDevTimeoutProducer);
          ok = false;
          break;
        }
        const uint32_t crow = smem_u32(sm.codes) + cs * (CODE_BYTES / CODE_SLOTS_DH) + krow * 128;
        const uint4 lo = lds128(crow + (((2 * box) ^ (krow & 7)) << 4));
        const uint4 hi = lds128(crow + (((2 * box + 1) ^ (krow & 7)) << 4));
        const int s = it % STAGES;
        if (!mbar_wait_warp(&sm.empty[s], ((it / STAGES) & 1) ^ 1, sm.abort_flag)) {
          if (lane == 0) raise_abort(sm, p.status, kDevTimeoutProducer);
          ok = false;
          break;
        }
        dq_store_row(smem_u32(sm.b(s)) + box * (64 * BK * 2) + krow * 128, krow & 7, lo, hi, sc, bi, qp_f32, valid);
        dq_signal_written(&sm.full[s], lane);
        if (lane == 0) mbar_arrive(&sm.cempty[cs]);   // after the codes were consumed (see ce_logits_kernel)
        ++it;
        advance(t_cur, kb_cur);
      }
    }
  } else if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmap_g);
      tma_prefetch_desc(&tmap_w);
      uint32_t it = 0;
      bool ok = true;
      for (int t = first_tile; t < total_tiles && ok; t += gridDim.x) {
        const int rb = t / p.num_nt;
        const int nt = t - rb * p.num_nt;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(&sm.empty[s], ((it / STAGES) & 1) ^ 1, sm.abort_flag)) {
            raise_abort(sm, p.status, kDevTimeoutProducer);
            ok = false;
            break;
          }
          if (QUANT) {
            // packed codes of the stage's 64 vocab rows x 256 hidden columns (tmap_w is the uint32 map here)
            const uint32_t cs = it % CODE_SLOTS_DH;
            if (!mbar_wait(&sm.cempty[cs], ((it / CODE_SLOTS_DH) & 1) ^ 1, sm.abort_flag)) {
              raise_abort(sm, p.status, kDevTimeoutProducer);
              ok = false;
              break;
            }
            mbar_arrive_expect_tx(&sm.cfull[cs], CODE_BYTES / CODE_SLOTS_DH);
            tma_load_2d(sm.codes + cs * (CODE_BYTES / CODE_SLOTS_DH), &tmap_w, &sm.cfull[cs], nt * (BN / 8),
                        p.wrow0 + kb * BK);
          }
          mbar_arrive_expect_tx(&sm.full[s], QUANT ? A_BYTES : STAGE_BYTES);
          tma_load_2d(sm.a(s), &tmap_g, &sm.full[s], kb * BK, rb * BM);
          // B tile: 64 vocab rows (K) x 256 hidden columns (N) as four [64 k][64 n] boxes.
          if (!QUANT) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sm.b(s) + j * (64 * BK * 2), &tmap_w, &sm.full[s], nt * BN + j * 64, p.wrow0 + kb * BK);
          }
        }
      }
      if (!ok) {
        producer_drain(sm, it);
        if (QUANT)
          for (uint32_t c = it > CODE_SLOTS_DH ? it - CODE_SLOTS_DH : 0; c < it; ++c)
            mbar_wait_drain(&sm.cfull[c % CODE_SLOTS_DH], (c / CODE_SLOTS_DH) & 1);
      }
    }
  } else if (warp == 1) {
    // whole-warp issue loop, one elected lane issues (see ce_logits_kernel)
    constexpr uint32_t idesc = make_idesc_bf16(BM, BN, 0, 1);  // B is MN-major
    constexpr uint32_t dhi = desc_hi_sw128(1024);
    uint32_t it = 0, tile = 0;
    bool ok = true;
    for (int t = first_tile; t < total_tiles && ok; t += gridDim.x, ++tile) {
      const uint32_t as = tile & 1;
      if (!mbar_wait_warp(&sm.tempty[as], ((tile >> 1) & 1) ^ 1, sm.abort_flag)) {
        if (lane == 0) raise_abort(sm, p.status, kDevTimeoutMma);
        break;
      }
      tc_fence_after_sync();
      const uint32_t d_tmem = tmem_base + as * BN;
      for (int kb = 0; kb < kblocks; ++kb, ++it) {
        const int s = it % STAGES;
        if (!mbar_wait_warp(&sm.full[s], (it / STAGES) & 1, sm.abort_flag)) {
          if (lane == 0) raise_abort(sm, p.status, kDevTimeoutMma);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t a_lo = desc_lo(smem_u32(sm.a(s)), 16);
        // 16 k rows of 128 B each per step; 64-column chunks are 8 KiB apart.
        const uint32_t b_lo = desc_lo(smem_u32(sm.b(s)), 64 * BK * 2);
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_ss_w(d_tmem, a_lo + k * 2, dhi, b_lo + k * 128, dhi, idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit(&sm.empty[s]);
        }
        __syncwarp();
      }
      if (ok && elect_one()) umma_commit(&sm.tfull[as]);
      __syncwarp();
    }
  } else {
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    uint32_t tile = 0;
    for (int t = first_tile; t < total_tiles; t += gridDim.x, ++tile) {
      const int rb = t / p.num_nt;
      const int nt = t - rb * p.num_nt;
      const uint32_t as = tile & 1;
      if (!mbar_wait_warp(&sm.tfull[as], (tile >> 1) & 1, sm.abort_flag)) {
        raise_abort(sm, p.status, kDevTimeoutEpilogue);
        break;
      }
      tc_fence_after_sync();
      const int row = rb * BM + row_in_tile;
      const bool row_ok = row < p.n_rows;
      const uint32_t taddr0 = tmem_base + as * BN + (static_cast<uint32_t>(quad * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = nt * BN + c * 32;
        if (col0 >= p.d_cols) break;
        uint32_t r[32];
        tmem_ld_x32(taddr0 + c * 32, r);
        tmem_wait_ld();
        tmem_regs_ready(r);
        if (row_ok) {
          const size_t off = static_cast<size_t>(row) * p.d_cols + col0;
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            if (col0 + j < p.d_cols) {  // d_cols is a multiple of 8
              float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                                     __uint_as_float(r[j + 3]));
              if (p.acc_in != nullptr) {
                const float4 o = *reinterpret_cast<const float4*>(p.acc_in + off + j);
                v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
              }
              if (p.acc_out != nullptr) *reinterpret_cast<float4*>(p.acc_out + off + j) = v;
              if (p.out_bf16 != nullptr) {
                uint2 w2 = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
                *reinterpret_cast<uint2*>(p.out_bf16 + off + j) = w2;
              }
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.tempty[as]);
    }
  }
  cta_teardown(sm, warp, tmem_base);
}

// -----------------------------------------------------------------------------------------
// dW_chunk = G^T hidden   (trainable dense head; core/chunked.py:84-85, K5 of the reference)
// -----------------------------------------------------------------------------------------
// Tile = 128 vocab rows x 256 hidden columns, contraction over the N tokens in 64-row blocks.
// Both operands are read MN-major straight from their row-major homes: A = G (N, chunk) as two
// [64 tokens][64 vocab columns] boxes per stage, B = hidden (N, D) as four [64 tokens][64 hidden
// columns] boxes.  Token rows past N are zero-filled by TMA.  Each vocab row belongs to exactly one
// chunk, so the fp32 accumulator is complete after one pass and is rounded once to bf16.
__global__ void __launch_bounds__(THREADS, 1)
ce_dw_kernel(const __grid_constant__ CUtensorMap tmap_g, const __grid_constant__ CUtensorMap tmap_h,
             const DwParams p) {
  extern __shared__ uint8_t smem_raw[];
  const SmemView sm = carve_smem(smem_raw);
  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);   // provably warp-uniform
  const int lane = threadIdx.x & 31;
  const uint32_t tmem_base = cta_setup(sm, warp);

  const int total_tiles = p.num_mt * p.num_nt;
  const int kblocks = (p.n_rows + BK - 1) / BK;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmap_g);
      tma_prefetch_desc(&tmap_h);
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const int nt = t / p.num_mt;
        const int mt = t - nt * p.num_mt;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(&sm.empty[s], ((it / STAGES) & 1) ^ 1, sm.abort_flag)) {
            raise_abort(sm, p.status, kDevTimeoutProducer);
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&sm.full[s], STAGE_BYTES);
#pragma unroll
          for (int j = 0; j < BM / 64; ++j)
            tma_load_2d(sm.a(s) + j * (64 * BK * 2), &tmap_g, &sm.full[s], mt * BM + j * 64, kb * BK);
#pragma unroll
          for (int j = 0; j < BN / 64; ++j)
            tma_load_2d(sm.b(s) + j * (64 * BK * 2), &tmap_h, &sm.full[s], nt * BN + j * 64, kb * BK);
        }
      }
      if (!ok) producer_drain(sm, it);
    }
  } else if (warp == 1) {
    // whole-warp issue loop, one elected lane issues (see ce_logits_kernel)
    constexpr uint32_t idesc = make_idesc_bf16(BM, BN, 1, 1);  // A and B are MN-major
    constexpr uint32_t dhi = desc_hi_sw128(1024);
    uint32_t it = 0, tile = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++tile) {
      const uint32_t as = tile & 1;
      if (!mbar_wait_warp(&sm.tempty[as], ((tile >> 1) & 1) ^ 1, sm.abort_flag)) {
        if (lane == 0) raise_abort(sm, p.status, kDevTimeoutMma);
        break;
      }
      tc_fence_after_sync();
      const uint32_t d_tmem = tmem_base + as * BN;
      for (int kb = 0; kb < kblocks; ++kb, ++it) {
        const int s = it % STAGES;
        if (!mbar_wait_warp(&sm.full[s], (it / STAGES) & 1, sm.abort_flag)) {
          if (lane == 0) raise_abort(sm, p.status, kDevTimeoutMma);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        // 16 token rows of 128 B per step; 64-column chunks are 8 KiB apart (both operands).
        const uint32_t a_lo = desc_lo(smem_u32(sm.a(s)), 64 * BK * 2);
        const uint32_t b_lo = desc_lo(smem_u32(sm.b(s)), 64 * BK * 2);
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_ss_w(d_tmem, a_lo + k * 128, dhi, b_lo + k * 128, dhi, idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit(&sm.empty[s]);
        }
        __syncwarp();
      }
      if (ok && elect_one()) umma_commit(&sm.tfull[as]);
      __syncwarp();
    }
  } else {
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    uint32_t tile = 0;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++tile) {
      const int nt = t / p.num_mt;
      const int mt = t - nt * p.num_mt;
      const uint32_t as = tile & 1;
      if (!mbar_wait_warp(&sm.tfull[as], (tile >> 1) & 1, sm.abort_flag)) {
        raise_abort(sm, p.status, kDevTimeoutEpilogue);
        break;
      }
      tc_fence_after_sync();
      const int row = mt * BM + row_in_tile;   // vocab row inside the chunk
      const bool row_ok = row < p.v_rows;
      const uint32_t taddr0 = tmem_base + as * BN + (static_cast<uint32_t>(quad * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = nt * BN + c * 32;
        if (col0 >= p.d_cols) break;
        uint32_t r[32];
        tmem_ld_x32(taddr0 + c * 32, r);
        tmem_wait_ld();
        tmem_regs_ready(r);
        if (row_ok) {
          __nv_bfloat16* dst = p.out + static_cast<size_t>(row) * p.d_cols + col0;
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (col0 + j < p.d_cols) {  // d_cols is a multiple of 8
              *reinterpret_cast<uint4*>(dst + j) = make_uint4(
                  pack_bf16x2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])),
                  pack_bf16x2(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3])),
                  pack_bf16x2(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5])),
                  pack_bf16x2(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7])));
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.tempty[as]);
    }
  }
  cta_teardown(sm, warp, tmem_base);
}

// -----------------------------------------------------------------------------------------
// Host-side scheduling
// -----------------------------------------------------------------------------------------
// Splits of the vocab-tile range: pick the count that minimises the busiest CTA's tile
// count under static round-robin, with a small per-unit cost for the partial writes.
// The search is O(splits * units) on the host, so results are memoised per shape.
int choose_splits(int num_rb, int num_vt, int ctas) {
  static std::mutex mu;
  static std::map<std::tuple<int, int, int>, int> memo;
  const auto key = std::make_tuple(num_rb, num_vt, ctas);
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = memo.find(key);
    if (it != memo.end()) return it->second;
  }
  int best = 1;
  double best_cost = 1e300;
  // More splits than ~8 waves of units buys nothing: cap the search.
  const int max_s = std::max(1, std::min(num_vt, std::max(1, 8 * ctas / std::max(1, num_rb) + 1)));
  std::vector<long long> load(ctas);
  for (int s = 1; s <= max_s; ++s) {
    std::fill(load.begin(), load.end(), 0);
    const long long units = static_cast<long long>(num_rb) * s;
    for (int split = 0; split < s; ++split) {
      const long long t0 = static_cast<long long>(split) * num_vt / s;
      const long long t1 = static_cast<long long>(split + 1) * num_vt / s;
      const long long u0 = static_cast<long long>(split) * num_rb;
      for (int rb = 0; rb < num_rb; ++rb) load[(u0 + rb) % ctas] += (t1 - t0);
    }
    const long long mx = *std::max_element(load.begin(), load.end());
    const double cost = static_cast<double>(mx) + 0.02 * static_cast<double>((units + ctas - 1) / ctas);
    if (cost < best_cost - 1e-9) {
      best_cost = cost;
      best = s;
    }
  }
  std::lock_guard<std::mutex> lock(mu);
  memo[key] = best;
  return best;
}

}  // namespace

static std::atomic<int> g_smem_configured[64];

static int configure_kernels() {
  int dev = 0;
  B200TP_CUDA_OK(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && g_smem_configured[dev].load(std::memory_order_acquire)) return B200TP_OK;
  B200TP_CUDA_OK(cudaFuncSetAttribute(ce_logits_kernel<MODE_FWD, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      SMEM_BYTES));
  B200TP_CUDA_OK(cudaFuncSetAttribute(ce_logits_kernel<MODE_BWD_G, false>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
  B200TP_CUDA_OK(cudaFuncSetAttribute(ce_logits_kernel<MODE_FWD, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      SMEM_BYTES_Q));
  B200TP_CUDA_OK(cudaFuncSetAttribute(ce_logits_kernel<MODE_BWD_G, true>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES_Q));
  B200TP_CUDA_OK(cudaFuncSetAttribute(ce_dh_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
  B200TP_CUDA_OK(cudaFuncSetAttribute(ce_dh_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES_Q));
  B200TP_CUDA_OK(cudaFuncSetAttribute(ce_dw_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
  if (dev >= 0 && dev < 64) g_smem_configured[dev].store(1, std::memory_order_release);
  return B200TP_OK;
}

int ce_tc_fwd_splits(int64_t n, int64_t v_rows) {
  const int num_rb = static_cast<int>(ceil_div(n, BM));
  const int num_vt = static_cast<int>(ceil_div(v_rows, BN));
  return choose_splits(num_rb, num_vt, sm_count());
}

// Tensor map of the weight operand: the dense bf16 matrix, or for a 4-bit head the map of its packed
// uint32 code words (box of `code_box_rows` rows x `code_box_words` words), which the producer copies
// into the code ring.
static int weight_map(CUtensorMap* out, const void* w, int64_t w_rows_total, int d, uint32_t box_rows,
                      uint32_t box_cols, const QuantHead* q, uint32_t code_box_rows, uint32_t code_box_words) {
  if (q != nullptr && q->wq != nullptr)
    return make_tmap_2d_u32(out, q->wq, w_rows_total, d / 8, d / 8, code_box_rows, code_box_words);
  return make_tmap_2d_bf16(out, w, w_rows_total, d, d, box_rows, box_cols);
}

static void fill_quant(LogitsParams& p, const QuantHead* q) {
  if (q == nullptr) return;
  p.wq = q->wq;
  p.scales = q->scales;
  p.biases = q->biases;
  p.qp_f32 = q->qp_f32;
  p.qvec = (!q->qp_f32 && p.k_dim % 512 == 0 && ((reinterpret_cast<uintptr_t>(q->scales) |
                                                  reinterpret_cast<uintptr_t>(q->biases)) & 15) == 0)
               ? 1
               : 0;
}

int ce_tc_launch_fwd(const void* hidden, const void* w, int64_t w_rows_total, int64_t n, int d, int64_t vrow0,
                     int64_t vrow1, int64_t vocab_id0, const int64_t* targets, int64_t ignore_index, int splits,
                     float* pm, float* ps, float* pt, const QuantHead* q, cudaStream_t stream, int* status) {
  int rc = configure_kernels();
  if (rc) return rc;
  CUtensorMap tmap_h, tmap_w;
  rc = make_tmap_2d_bf16(&tmap_h, hidden, n, d, d, BM, BK);
  if (rc) return rc;
  rc = weight_map(&tmap_w, w, w_rows_total, d, BN, BK, q, BN, 16);
  if (rc) return rc;
  LogitsParams p{};
  p.n_rows = static_cast<int>(n);
  p.k_dim = d;
  p.vrow0 = static_cast<int>(vrow0);
  p.vrow1 = static_cast<int>(vrow1);
  p.vocab_id0 = vocab_id0;
  p.num_rb = static_cast<int>(ceil_div(n, BM));
  p.num_vt = static_cast<int>(ceil_div(vrow1 - vrow0, BN));
  p.splits = splits;
  p.targets = reinterpret_cast<const long long*>(targets);
  p.ignore_index = ignore_index;
  p.pm = pm;
  p.ps = ps;
  p.pt = pt;
  p.status = status;
  fill_quant(p, q);
  const int grid = std::min<long long>(sm_count(), static_cast<long long>(p.num_rb) * splits);
  if (p.wq != nullptr)
    ce_logits_kernel<MODE_FWD, true><<<grid, THREADS_Q, SMEM_BYTES_Q, stream>>>(tmap_h, tmap_w, p);
  else
    ce_logits_kernel<MODE_FWD, false><<<grid, THREADS, SMEM_BYTES, stream>>>(tmap_h, tmap_w, p);
  B200TP_CUDA_OK(cudaGetLastError());
  return B200TP_OK;
}

int ce_tc_launch_bwd_g(const void* hidden, const void* w, int64_t w_rows_total, int64_t n, int d, int64_t vrow0,
                       int64_t vrow1, int64_t vocab_id0, const int64_t* targets, int64_t ignore_index,
                       const float* lse, const float* ct, void* g, int ldg, const QuantHead* q, cudaStream_t stream,
                       int* status) {
  int rc = configure_kernels();
  if (rc) return rc;
  CUtensorMap tmap_h, tmap_w;
  rc = make_tmap_2d_bf16(&tmap_h, hidden, n, d, d, BM, BK);
  if (rc) return rc;
  rc = weight_map(&tmap_w, w, w_rows_total, d, BN, BK, q, BN, 16);
  if (rc) return rc;
  LogitsParams p{};
  p.n_rows = static_cast<int>(n);
  p.k_dim = d;
  p.vrow0 = static_cast<int>(vrow0);
  p.vrow1 = static_cast<int>(vrow1);
  p.vocab_id0 = vocab_id0;
  p.num_rb = static_cast<int>(ceil_div(n, BM));
  p.num_vt = static_cast<int>(ceil_div(vrow1 - vrow0, BN));
  // One unit per (row block, vocab tile group): there is no cross-tile state in this
  // mode, so split as finely as balance asks for.
  p.splits = choose_splits(p.num_rb, p.num_vt, sm_count());
  p.targets = reinterpret_cast<const long long*>(targets);
  p.ignore_index = ignore_index;
  p.lse = lse;
  p.ct = ct;
  p.g = reinterpret_cast<__nv_bfloat16*>(g);
  p.ldg = ldg;
  p.status = status;
  fill_quant(p, q);
  const int grid = std::min<long long>(sm_count(), static_cast<long long>(p.num_rb) * p.splits);
  if (p.wq != nullptr)
    ce_logits_kernel<MODE_BWD_G, true><<<grid, THREADS_Q, SMEM_BYTES_Q, stream>>>(tmap_h, tmap_w, p);
  else
    ce_logits_kernel<MODE_BWD_G, false><<<grid, THREADS, SMEM_BYTES, stream>>>(tmap_h, tmap_w, p);
  B200TP_CUDA_OK(cudaGetLastError());
  return B200TP_OK;
}

int ce_tc_dh_tiles(int64_t n, int d) {
  return static_cast<int>(ceil_div(n, BM) * ceil_div(d, BN));
}

int ce_tc_dh_rows_done(int64_t n, int d, int tiles_done) {
  const int num_nt = static_cast<int>(ceil_div(d, BN));
  if (tiles_done >= ce_tc_dh_tiles(n, d)) return static_cast<int>(n);
  return static_cast<int>(std::min<int64_t>(n, static_cast<int64_t>(tiles_done / num_nt) * BM));
}

int ce_tc_launch_dh(const void* g, int ldg, int k_total, int64_t n, const void* w, int64_t w_rows_total, int d,
                    int64_t wrow0, const float* acc_in, float* acc_out, void* out_bf16, int tile0, int tile1,
                    const QuantHead* q, cudaStream_t stream, int* status) {
  int rc = configure_kernels();
  if (rc) return rc;
  CUtensorMap tmap_g, tmap_w;
  rc = make_tmap_2d_bf16(&tmap_g, g, n, k_total, ldg, BM, BK);
  if (rc) return rc;
  rc = weight_map(&tmap_w, w, w_rows_total, d, /*box_rows=*/BK, /*box_cols=*/64, q, BK, BN / 8);
  if (rc) return rc;
  DhParams p{};
  p.n_rows = static_cast<int>(n);
  p.d_cols = d;
  p.k_total = k_total;
  p.wrow0 = static_cast<int>(wrow0);
  p.num_rb = static_cast<int>(ceil_div(n, BM));
  p.num_nt = static_cast<int>(ceil_div(d, BN));
  p.acc_in = acc_in;
  p.acc_out = acc_out;
  p.out_bf16 = reinterpret_cast<__nv_bfloat16*>(out_bf16);
  p.status = status;
  const int total = p.num_rb * p.num_nt;
  p.tile0 = tile0 < 0 ? 0 : tile0;
  p.tile1 = tile1 < 0 ? total : std::min(tile1, total);
  p.w_rows = static_cast<int>(w_rows_total);
  if (q != nullptr) {
    p.wq = q->wq;
    p.scales = q->scales;
    p.biases = q->biases;
    p.qp_f32 = q->qp_f32;
  }
  if (p.tile1 <= p.tile0) return B200TP_OK;
  const int grid = std::min<long long>(sm_count(), p.tile1 - p.tile0);
  if (p.wq != nullptr)
    ce_dh_kernel<true><<<grid, THREADS_Q, SMEM_BYTES_Q, stream>>>(tmap_g, tmap_w, p);
  else
    ce_dh_kernel<false><<<grid, THREADS, SMEM_BYTES, stream>>>(tmap_g, tmap_w, p);
  B200TP_CUDA_OK(cudaGetLastError());
  return B200TP_OK;
}

int ce_tc_launch_dw(const void* g, int ldg, int64_t v_rows, int64_t n, const void* hidden, int d, void* d_weight_block,
                    cudaStream_t stream, int* status) {
  int rc = configure_kernels();
  if (rc) return rc;
  CUtensorMap tmap_g, tmap_h;
  // both maps: 64 token rows x 64 columns per box
  rc = make_tmap_2d_bf16(&tmap_g, g, n, ldg, ldg, /*box_rows=*/BK, /*box_cols=*/64);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tmap_h, hidden, n, d, d, /*box_rows=*/BK, /*box_cols=*/64);
  if (rc) return rc;
  DwParams p{};
  p.n_rows = static_cast<int>(n);
  p.d_cols = d;
  p.v_rows = static_cast<int>(v_rows);
  p.num_mt = static_cast<int>(ceil_div(v_rows, BM));
  p.num_nt = static_cast<int>(ceil_div(d, BN));
  p.out = reinterpret_cast<__nv_bfloat16*>(d_weight_block);
  p.status = status;
  const int grid = std::min<long long>(sm_count(), static_cast<long long>(p.num_mt) * p.num_nt);
  ce_dw_kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(tmap_g, tmap_h, p);
  B200TP_CUDA_OK(cudaGetLastError());
  return B200TP_OK;
}

}  // namespace b200tp
