// C ABI of the fused linear cross-entropy: argument checks, workspace carving and the
// per-chunk launch sequences of the two implementations (tcgen05 and SIMT).
#include <string>

#include "common.h"
#include "linear_ce_simt.h"
#include "linear_ce_tc.h"

namespace b200tp {
const char* last_error_cstr();

namespace {

// Default upper bound on the vocab rows per backward chunk: kTcChunkRowsMax, fewer when N is so large that
// the (N, chunk) bf16 matrix of g would exceed kTcScratchBytes.  Measured at N=8192, D=4096, V=151936
// (backward alone, ms / workspace): bound 4096 20.0 / 192 MB, 8192 18.3 / 256 MB, 16384 18.2 / 368 MB,
// 32768 17.5 / 604 MB, larger no faster.  Inside the power-capped forward + backward step the last gain
// disappears (24.73 against 24.81 ms per step), so the default stays at the smaller scratch.
constexpr int64_t kTcChunkRowsMax = 16384;
constexpr int64_t kTcChunkRowsMin = 2048;
constexpr int64_t kTcScratchBytes = 512ll << 20;
constexpr int64_t kSimtChunkRows = 4096;  // vocab rows per SIMT chunk

// Vocab rows per tensor-core backward chunk for a shard of `v` rows.  The bound (the default above, or what
// the caller asked for in `reserved`) trades scratch for launches: the (N, chunk) bf16 matrix of g is the
// backward's main workspace.  The rows are spread evenly over the fewest chunks the bound allows (a
// short last chunk would keep the second GEMM's contraction too short to hide its fp32 accumulator
// round trip).
constexpr int kReservedInline = 0x10000;    // 4-bit head: expand inside the kernels whatever the row count
constexpr int kReservedChunked = 0x20000;   // 4-bit head: dequantise chunk by chunk whatever the row count
constexpr int64_t kInlineMaxRows = 512;     // default: the forward expands in the kernel up to this many rows of hidden

int64_t tc_chunk_rows(const b200tp_ce_args* a, int64_t* num_chunks) {
  int64_t bound = static_cast<int64_t>(a->reserved & 0xFFFF) * kCeTileCols;
  if (bound <= 0) {
    const int64_t fit = kTcScratchBytes / (2 * std::max<int64_t>(a->n, 1)) / kCeTileCols * kCeTileCols;
    bound = std::min(kTcChunkRowsMax, std::max(kTcChunkRowsMin, fit));
  }
  const int64_t nc = ceil_div(a->v_local, bound);
  *num_chunks = nc;
  return static_cast<int64_t>(align_up(static_cast<size_t>(ceil_div(a->v_local, nc)), kCeTileCols));
}

struct Bump {
  char* base;
  size_t off = 0;
  explicit Bump(void* p) : base(static_cast<char*>(p)) {}
  template <typename T>
  T* take(size_t count) {
    off = align_up(off, 256);
    T* p = base ? reinterpret_cast<T*>(base + off) : nullptr;
    off += count * sizeof(T);
    return p;
  }
};

int check_args(const b200tp_ce_args* a) {
  if (a == nullptr) return fail(B200TP_ERR_LOSS_INPUT, "args is null");
  if (a->n <= 0) return fail(B200TP_ERR_LOSS_INPUT, "hidden must have at least one row (n=" + std::to_string(a->n) + ")");
  if (a->d <= 0 || a->v_local <= 0) return fail(B200TP_ERR_LOSS_INPUT, "d and v_local must be positive");
  if (a->n > (1ll << 30) || a->v_local > (1ll << 30)) return fail(B200TP_ERR_LOSS_INPUT, "n / v_local too large");
  if (a->dtype != B200TP_F32 && a->dtype != B200TP_BF16)
    return fail(B200TP_ERR_UNSUPPORTED_HEAD, "only fp32 / bf16 hidden dtypes are supported");
  if (a->hidden == nullptr || a->targets == nullptr) return fail(B200TP_ERR_LOSS_INPUT, "hidden / targets is null");
  if (a->quant_bits == 0) {
    if (a->weight == nullptr) return fail(B200TP_ERR_LOSS_INPUT, "dense head without a weight pointer");
  } else if (a->quant_bits == 4) {
    if (a->group_size != 64)
      return fail(B200TP_ERR_UNSUPPORTED_HEAD, "only group_size=64 quantized heads are supported (got " +
                                                   std::to_string(a->group_size) + ")");
    if (a->d % 64 != 0)
      return fail(B200TP_ERR_UNSUPPORTED_HEAD, "a quantized head needs a hidden size that is a multiple of 64");
    if (a->w_q == nullptr || a->scales == nullptr || a->biases == nullptr)
      return fail(B200TP_ERR_LOSS_INPUT, "quantized head with a null w_q / scales / biases pointer");
    if (a->qparam_dtype != B200TP_F32 && a->qparam_dtype != B200TP_BF16)
      return fail(B200TP_ERR_UNSUPPORTED_HEAD, "scales / biases must be fp32 or bf16");
  } else {
    return fail(B200TP_ERR_UNSUPPORTED_HEAD,
                "only 4-bit quantized heads are supported (got bits=" + std::to_string(a->quant_bits) + ")");
  }
  if (a->impl != B200TP_IMPL_AUTO && a->impl != B200TP_IMPL_TC && a->impl != B200TP_IMPL_SIMT)
    return fail(B200TP_ERR_LOSS_INPUT, "unknown impl selector");
  if (a->reserved < 0 || (a->reserved & ~(0xFFFF | kReservedInline | kReservedChunked)) != 0 ||
      (a->reserved & (kReservedInline | kReservedChunked)) == (kReservedInline | kReservedChunked))
    return fail(B200TP_ERR_LOSS_INPUT,
                "reserved holds the backward chunk bound (low 16 bits, units of 256 vocab rows) and at most one of "
                "the 4-bit dequantisation selectors 0x10000 / 0x20000");
  return B200TP_OK;
}

// Where a 4-bit head is expanded on the tensor-core path.
//   in the kernels: the weight operand never exists in global memory, but every CTA that meets a weight
//     tile expands it again, i.e. once per 128 rows of hidden: ALU work that grows with N and, past a few
//     row blocks, exceeds what the tensor pipe leaves idle (measured at N=8192: 2.2x the dense forward);
//   chunk by chunk into a bf16 scratch (one pass over the codes per GEMM pass, 0.06 ms per 16384 x 4096
//     chunk) followed by the dense kernels: the cheaper form for training-sized batches.
// Default, from timings at D=4096, V=151936 (in-kernel / chunked, ms): forward 0.36 / 1.25 at N=128,
// 1.02 / 1.25 at 512, 1.93 / 1.56 at 1024 -- in the kernel up to kInlineMaxRows rows, with no weight
// scratch at all; backward 3.2 / 1.9 at N=128, 3.8 / 2.1 at 512 -- always chunked: with few row blocks
// the d_hidden GEMM has only D / 256 tiles, so a handful of CTAs would each expand their 256 columns of
// the whole head, while the dequantisation kernel spreads the same work over every SM.  `reserved`
// can force either form in both directions (in-kernel needs no weight scratch).  The in-kernel path
// needs a 16-byte aligned w_q (TMA).
bool quant_inline(const b200tp_ce_args* a, bool backward) {
  if (a->quant_bits != 4 || (reinterpret_cast<uintptr_t>(a->w_q) & 15) != 0) return false;
  if (a->reserved & kReservedInline) return true;
  if (a->reserved & kReservedChunked) return false;
  return !backward && a->n <= kInlineMaxRows;
}

QuantHead quant_head(const b200tp_ce_args* a, bool backward) {
  QuantHead q{};
  if (quant_inline(a, backward)) {
    q.wq = a->w_q;
    q.scales = a->scales;
    q.biases = a->biases;
    q.qp_f32 = a->qparam_dtype == B200TP_F32 ? 1 : 0;
  }
  return q;
}

// 1 = tcgen05, 2 = SIMT, negative = refusal already recorded
int pick_impl(const b200tp_ce_args* a) {
  const bool tc_ok = a->dtype == B200TP_BF16 && a->d % 8 == 0;
  if (a->impl == B200TP_IMPL_SIMT) return 2;
  if (a->impl == B200TP_IMPL_TC) {
    if (!tc_ok) {
      fail(B200TP_ERR_UNSUPPORTED_HEAD,
           "the tensor-core path needs bf16 operands and a hidden size that is a multiple of 8; use impl=simt");
      return -1;
    }
    if ((a->reserved & kReservedInline) && !quant_inline(a, false)) {
      fail(B200TP_ERR_UNSUPPORTED_HEAD, "in-kernel dequantisation needs a 4-bit head with a 16-byte aligned w_q");
      return -1;
    }
    return 1;
  }
  return tc_ok ? 1 : 2;
}

size_t elem_size(int dtype) { return dtype == B200TP_BF16 ? 2 : 4; }

struct FwdPlan {
  int impl;
  int64_t chunk;        // vocab rows per launch (tc dense: all)
  int64_t num_chunks;
  int64_t total_splits; // tc only
  // workspace pointers
  float* pm; float* ps; float* pt;
  void* deq;
  float* logits;
  size_t bytes;
};

FwdPlan plan_fwd(const b200tp_ce_args* a, void* ws) {
  FwdPlan p{};
  p.impl = pick_impl(a);
  if (p.impl < 0) return p;
  Bump b(ws);
  if (p.impl == 1) {
    if (a->quant_bits == 0 || quant_inline(a, false)) {
      // one launch over the whole shard (a 4-bit head is expanded inside the kernel, tile by tile)
      p.chunk = a->v_local;
      p.num_chunks = 1;
      p.total_splits = ce_tc_fwd_splits(a->n, a->v_local);
    } else {
      // 4-bit head, chunked: dequantise a chunk of vocab rows, run the dense kernel over it
      p.chunk = tc_chunk_rows(a, &p.num_chunks);
      p.total_splits = 0;
      for (int64_t c = 0; c < p.num_chunks; ++c) {
        const int64_t w = std::min<int64_t>(p.chunk, a->v_local - c * p.chunk);
        p.total_splits += ce_tc_fwd_splits(a->n, w);
      }
      p.deq = b.take<char>(static_cast<size_t>(p.chunk) * a->d * 2);
    }
    p.pm = b.take<float>(static_cast<size_t>(p.total_splits) * a->n);
    p.ps = b.take<float>(static_cast<size_t>(p.total_splits) * a->n);
    p.pt = b.take<float>(static_cast<size_t>(p.total_splits) * a->n);
  } else {
    p.chunk = std::min<int64_t>(kSimtChunkRows, a->v_local);
    p.num_chunks = ceil_div(a->v_local, p.chunk);
    p.logits = b.take<float>(static_cast<size_t>(a->n) * p.chunk);
    if (a->quant_bits != 0) p.deq = b.take<char>(static_cast<size_t>(p.chunk) * a->d * elem_size(a->dtype));
  }
  p.bytes = align_up(b.off, 256);
  return p;
}

struct BwdPlan {
  int impl;
  int64_t chunk, num_chunks;
  int ldg;
  void* g;        // tc: bf16 (n, ldg)
  float* logits;  // simt: f32 (n, chunk)
  float* acc;     // f32 (n, d) when the output is bf16 and must be accumulated in fp32
  void* deq;
  size_t bytes;
};

BwdPlan plan_bwd(const b200tp_ce_args* a, int out_dtype, void* ws) {
  BwdPlan p{};
  p.impl = pick_impl(a);
  if (p.impl < 0) return p;
  Bump b(ws);
  if (p.impl == 1) {
    p.chunk = tc_chunk_rows(a, &p.num_chunks);
    p.ldg = static_cast<int>(p.chunk);
    p.g = b.take<char>(static_cast<size_t>(a->n) * p.ldg * 2);
    if (out_dtype == B200TP_BF16 && p.num_chunks > 1) p.acc = b.take<float>(static_cast<size_t>(a->n) * a->d);
    if (a->quant_bits != 0 && !quant_inline(a, true)) p.deq = b.take<char>(static_cast<size_t>(p.chunk) * a->d * 2);
  } else {
    p.chunk = std::min<int64_t>(kSimtChunkRows, a->v_local);
    p.num_chunks = ceil_div(a->v_local, p.chunk);
    p.logits = b.take<float>(static_cast<size_t>(a->n) * p.chunk);
    if (out_dtype == B200TP_BF16) p.acc = b.take<float>(static_cast<size_t>(a->n) * a->d);
    if (a->quant_bits != 0) p.deq = b.take<char>(static_cast<size_t>(p.chunk) * a->d * elem_size(a->dtype));
  }
  p.bytes = align_up(b.off, 256);
  return p;
}

int check_workspace(void* ws, size_t have, size_t need) {
  if (need == 0) return B200TP_OK;
  if (ws == nullptr) return fail(B200TP_ERR_WORKSPACE, "workspace is null but " + std::to_string(need) + " bytes are needed");
  if ((reinterpret_cast<uintptr_t>(ws) & 255) != 0) return fail(B200TP_ERR_WORKSPACE, "workspace must be 256-byte aligned");
  if (have < need)
    return fail(B200TP_ERR_WORKSPACE,
                "workspace too small: have " + std::to_string(have) + ", need " + std::to_string(need) + " bytes");
  return B200TP_OK;
}

}  // namespace
}  // namespace b200tp

using namespace b200tp;

extern "C" {

size_t b200tp_linear_ce_fwd_workspace_bytes(const b200tp_ce_args* a) {
  if (check_args(a) != B200TP_OK) return 0;
  FwdPlan p = plan_fwd(a, nullptr);
  return p.impl < 0 ? 0 : p.bytes;
}

int b200tp_linear_ce_fwd(const b200tp_ce_args* a, float* row_max, float* row_sumexp, float* tgt_logit, float* lse,
                         float* nll, void* workspace, size_t workspace_bytes, void* stream_v, int* status) {
  int rc = check_args(a);
  if (rc) return rc;
  if (row_max == nullptr || row_sumexp == nullptr || tgt_logit == nullptr)
    return fail(B200TP_ERR_LOSS_INPUT, "row_max / row_sumexp / tgt_logit outputs are required");
  rc = require_sm100();
  if (rc) return rc;
  FwdPlan p = plan_fwd(a, workspace);
  if (p.impl < 0) return B200TP_ERR_UNSUPPORTED_HEAD;
  rc = check_workspace(workspace, workspace_bytes, p.bytes);
  if (rc) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

  if (p.impl == 1) {
    if (p.deq == nullptr) {
      const int splits = static_cast<int>(p.total_splits);
      const QuantHead q = quant_head(a, false);
      rc = ce_tc_launch_fwd(a->hidden, a->weight, a->v_local, a->n, a->d, 0, a->v_local, a->v_offset, a->targets,
                            a->ignore_index, splits, p.pm, p.ps, p.pt, &q, stream, status);
      if (rc) return rc;
    } else {
      int64_t slot = 0;
      for (int64_t c = 0; c < p.num_chunks; ++c) {
        const int64_t r0 = c * p.chunk;
        const int64_t w = std::min<int64_t>(p.chunk, a->v_local - r0);
        rc = launch_dequant_int4(a->w_q, a->scales, a->biases, a->qparam_dtype, r0, w, a->d, a->group_size, p.deq,
                                 B200TP_BF16, stream);
        if (rc) return rc;
        const int splits = ce_tc_fwd_splits(a->n, w);
        rc = ce_tc_launch_fwd(a->hidden, p.deq, w, a->n, a->d, 0, w, a->v_offset + r0, a->targets, a->ignore_index,
                              splits, p.pm + slot * a->n, p.ps + slot * a->n, p.pt + slot * a->n, nullptr, stream,
                              status);
        if (rc) return rc;
        slot += splits;
      }
    }
    return launch_combine(p.pm, p.ps, p.pt, a->n, static_cast<int>(p.total_splits), a->n, a->targets,
                          a->ignore_index, row_max, row_sumexp, tgt_logit, lse, nll, stream);
  }

  // SIMT: running triples live directly in the caller's output arrays.
  for (int64_t c = 0; c < p.num_chunks; ++c) {
    const int64_t r0 = c * p.chunk;
    const int64_t w = std::min<int64_t>(p.chunk, a->v_local - r0);
    const void* wc;
    if (a->quant_bits == 0) {
      wc = static_cast<const char*>(a->weight) + static_cast<size_t>(r0) * a->d * elem_size(a->dtype);
    } else {
      rc = launch_dequant_int4(a->w_q, a->scales, a->biases, a->qparam_dtype, r0, w, a->d, a->group_size, p.deq,
                               a->dtype, stream);
      if (rc) return rc;
      wc = p.deq;
    }
    rc = ce_simt_fwd_chunk(a->hidden, wc, a->dtype, a->n, a->d, w, a->v_offset + r0, a->targets, a->ignore_index,
                           p.logits, row_max, row_sumexp, tgt_logit, c == 0 ? 1 : 0, stream);
    if (rc) return rc;
  }
  return launch_combine(row_max, row_sumexp, tgt_logit, a->n, 1, a->n, a->targets, a->ignore_index, nullptr, nullptr,
                        tgt_logit, lse, nll, stream);
}

int b200tp_linear_ce_combine(const float* parts, int32_t num_parts, int64_t n, const int64_t* targets,
                             int64_t ignore_index, float* lse, float* nll, float* tgt_logit, void* stream) {
  if (parts == nullptr || num_parts <= 0 || n <= 0)
    return fail(B200TP_ERR_LOSS_INPUT, "combine needs at least one part and one row");
  return launch_combine(parts, parts + n, parts + 2 * n, 3 * n, num_parts, n, targets, ignore_index, nullptr, nullptr,
                        tgt_logit, lse, nll, static_cast<cudaStream_t>(stream));
}

int b200tp_linear_ce_reduce(const float* nll, const int64_t* targets, int64_t n, int64_t ignore_index, float* out3,
                            void* stream) {
  if (nll == nullptr || out3 == nullptr || n <= 0)
    return fail(B200TP_ERR_LOSS_INPUT, "reduce needs nll, an output triple and at least one row");
  return launch_loss_reduce(nll, targets, n, ignore_index, out3, static_cast<cudaStream_t>(stream));
}

int b200tp_linear_ce_cotangent(const int64_t* targets, int64_t n, int64_t ignore_index, const float* upstream,
                               const float* count, float* cotangent, void* stream) {
  if (upstream == nullptr || cotangent == nullptr || n <= 0)
    return fail(B200TP_ERR_LOSS_INPUT, "cotangent needs the upstream scalar, an output vector and at least one row");
  return launch_loss_cotangent(targets, n, ignore_index, upstream, count, cotangent,
                               static_cast<cudaStream_t>(stream));
}

size_t b200tp_linear_ce_bwd_workspace_bytes(const b200tp_ce_args* a, int32_t d_hidden_dtype) {
  if (check_args(a) != B200TP_OK) return 0;
  BwdPlan p = plan_bwd(a, d_hidden_dtype, nullptr);
  return p.impl < 0 ? 0 : p.bytes;
}

// Stages: the tensor-core backward can be issued in `num_stages` calls.  Stage 0 launches everything
// up to and including the first slab of the LAST chunk's d_hidden GEMM; stage s > 0 launches slab s of
// it.  The slabs are whole waves of the row-block-major tile order, so their launches cost what the
// single launch costs, and the leading `*rows_done` rows of d_hidden are final once a stage's work has
// run.  num_stages == 1 is the plain backward.
static int bwd_impl(const b200tp_ce_args* a, const float* lse, const float* cotangent, void* d_hidden,
                    int32_t d_hidden_dtype, int32_t accumulate, void* d_weight, int num_stages, int stage,
                    int64_t* rows_done, void* workspace, size_t workspace_bytes, void* stream_v, int* status) {
  int rc = check_args(a);
  if (rc) return rc;
  if (d_weight != nullptr && a->quant_bits != 0)
    return fail(B200TP_ERR_UNSUPPORTED_HEAD, "a quantized head is frozen: it has no d_weight");
  if (lse == nullptr || cotangent == nullptr || d_hidden == nullptr)
    return fail(B200TP_ERR_LOSS_INPUT, "lse / cotangent / d_hidden is null");
  if (d_hidden_dtype != B200TP_F32 && d_hidden_dtype != a->dtype)
    return fail(B200TP_ERR_LOSS_INPUT, "d_hidden dtype must be the hidden dtype or fp32");
  if (accumulate && d_hidden_dtype != B200TP_F32)
    return fail(B200TP_ERR_LOSS_INPUT, "accumulate is only defined for an fp32 d_hidden");
  if (num_stages < 1 || num_stages > 64 || stage < 0 || stage >= num_stages)
    return fail(B200TP_ERR_LOSS_INPUT, "stage must lie in [0, num_stages) with 1 <= num_stages <= 64");
  rc = require_sm100();
  if (rc) return rc;
  BwdPlan p = plan_bwd(a, d_hidden_dtype, workspace);
  if (p.impl < 0) return B200TP_ERR_UNSUPPORTED_HEAD;
  rc = check_workspace(workspace, workspace_bytes, p.bytes);
  if (rc) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const bool out_f32 = d_hidden_dtype == B200TP_F32;

  if (p.impl == 1) {
    const QuantHead q = quant_head(a, true);
    // slab `stage` of the last chunk's d_hidden tiles: whole waves of the persistent grid
    const int tiles = ce_tc_dh_tiles(a->n, a->d);
    const int ctas = sm_count();
    const int waves = static_cast<int>(ceil_div(tiles, ctas));
    auto slab_begin = [&](int s) { return std::min<int64_t>(tiles, static_cast<int64_t>(ctas) * (waves * s / num_stages)); };
    const int tile0 = static_cast<int>(slab_begin(stage));
    const int tile1 = stage + 1 == num_stages ? tiles : static_cast<int>(slab_begin(stage + 1));
    if (rows_done != nullptr) *rows_done = ce_tc_dh_rows_done(a->n, a->d, tile1);
    for (int64_t c = stage == 0 ? 0 : p.num_chunks - 1; c < p.num_chunks; ++c) {
      const int64_t r0 = c * p.chunk;
      const int64_t w = std::min<int64_t>(p.chunk, a->v_local - r0);
      const bool first = c == 0, last = c == p.num_chunks - 1;
      // weight operand of this chunk: rows [row0, row0 + w) of `wmat` (the dense head, the packed head, or
      // the chunk's dequantised copy, which stays valid for every stage's d_hidden launches of the chunk)
      const void* wmat = a->weight;
      int64_t wrows = a->v_local, row0 = r0, vocab_id0 = a->v_offset;
      const QuantHead* qp = &q;
      if (p.deq != nullptr) {
        if (stage == 0) {
          rc = launch_dequant_int4(a->w_q, a->scales, a->biases, a->qparam_dtype, r0, w, a->d, a->group_size, p.deq,
                                   B200TP_BF16, stream);
          if (rc) return rc;
        }
        wmat = p.deq;
        wrows = w;
        row0 = 0;
        vocab_id0 = a->v_offset + r0;
        qp = nullptr;
      }
      if (stage == 0) {
        rc = ce_tc_launch_bwd_g(a->hidden, wmat, wrows, a->n, a->d, row0, row0 + w, vocab_id0, a->targets,
                                a->ignore_index, lse, cotangent, p.g, p.ldg, qp, stream, status);
        if (rc) return rc;
      }
      const int k_total = static_cast<int>(align_up(w, kCeTileCols));
      const float* acc_in;
      float* acc_out;
      void* out_bf16;
      if (out_f32) {
        acc_in = (first && !accumulate) ? nullptr : static_cast<const float*>(d_hidden);
        acc_out = static_cast<float*>(d_hidden);
        out_bf16 = nullptr;
      } else {
        acc_in = first ? nullptr : p.acc;
        acc_out = last ? nullptr : p.acc;
        out_bf16 = last ? d_hidden : nullptr;
      }
      rc = ce_tc_launch_dh(p.g, p.ldg, k_total, a->n, wmat, wrows, a->d, row0, acc_in, acc_out, out_bf16,
                           last ? tile0 : -1, last ? tile1 : -1, qp, stream, status);
      if (rc) return rc;
      if (d_weight != nullptr) {
        void* block = static_cast<char*>(d_weight) + static_cast<size_t>(r0) * a->d * elem_size(a->dtype);
        rc = ce_tc_launch_dw(p.g, p.ldg, w, a->n, a->hidden, a->d, block, stream, status);
        if (rc) return rc;
      }
    }
    return B200TP_OK;
  }

  // CUDA-core path: not staged (everything runs in stage 0)
  if (rows_done != nullptr) *rows_done = a->n;
  if (stage > 0) return B200TP_OK;
  float* acc = out_f32 ? static_cast<float*>(d_hidden) : p.acc;
  for (int64_t c = 0; c < p.num_chunks; ++c) {
    const int64_t r0 = c * p.chunk;
    const int64_t w = std::min<int64_t>(p.chunk, a->v_local - r0);
    const void* wc;
    if (a->quant_bits == 0) {
      wc = static_cast<const char*>(a->weight) + static_cast<size_t>(r0) * a->d * elem_size(a->dtype);
    } else {
      rc = launch_dequant_int4(a->w_q, a->scales, a->biases, a->qparam_dtype, r0, w, a->d, a->group_size, p.deq,
                               a->dtype, stream);
      if (rc) return rc;
      wc = p.deq;
    }
    const int acc_flag = (c > 0 || (out_f32 && accumulate)) ? 1 : 0;
    rc = ce_simt_bwd_chunk(a->hidden, wc, a->dtype, a->n, a->d, w, a->v_offset + r0, a->targets, a->ignore_index, lse,
                           cotangent, p.logits, acc, acc_flag, stream);
    if (rc) return rc;
    if (d_weight != nullptr) {
      void* block = static_cast<char*>(d_weight) + static_cast<size_t>(r0) * a->d * elem_size(a->dtype);
      rc = ce_simt_dw_chunk(p.logits, w, a->hidden, a->dtype, a->n, a->d, block, stream);
      if (rc) return rc;
    }
  }
  if (!out_f32) return launch_cast_f32_to_bf16(acc, d_hidden, a->n * a->d, stream);
  return B200TP_OK;
}

int b200tp_linear_ce_bwd(const b200tp_ce_args* a, const float* lse, const float* cotangent, void* d_hidden,
                         int32_t d_hidden_dtype, int32_t accumulate, void* workspace, size_t workspace_bytes,
                         void* stream_v, int* status) {
  return bwd_impl(a, lse, cotangent, d_hidden, d_hidden_dtype, accumulate, nullptr, 1, 0, nullptr, workspace,
                  workspace_bytes, stream_v, status);
}

int b200tp_linear_ce_bwd_stage(const b200tp_ce_args* a, const float* lse, const float* cotangent, void* d_hidden,
                               int32_t d_hidden_dtype, int32_t accumulate, int32_t num_stages, int32_t stage,
                               int64_t* rows_done, void* workspace, size_t workspace_bytes, void* stream_v,
                               int* status) {
  return bwd_impl(a, lse, cotangent, d_hidden, d_hidden_dtype, accumulate, nullptr, num_stages, stage, rows_done,
                  workspace, workspace_bytes, stream_v, status);
}

int b200tp_linear_ce_bwd_train(const b200tp_ce_args* a, const float* lse, const float* cotangent, void* d_hidden,
                               int32_t d_hidden_dtype, int32_t accumulate, void* d_weight, void* workspace,
                               size_t workspace_bytes, void* stream_v, int* status) {
  if (d_weight == nullptr) return fail(B200TP_ERR_LOSS_INPUT, "d_weight is null");
  return bwd_impl(a, lse, cotangent, d_hidden, d_hidden_dtype, accumulate, d_weight, 1, 0, nullptr, workspace,
                  workspace_bytes, stream_v, status);
}

int b200tp_dequant_int4(const uint32_t* w_q, const void* scales, const void* biases, int32_t qparam_dtype, int64_t row0,
                        int64_t rows, int32_t d, int32_t group_size, void* out, int32_t out_dtype, void* stream) {
  if (w_q == nullptr || scales == nullptr || biases == nullptr || out == nullptr)
    return fail(B200TP_ERR_LOSS_INPUT, "null pointer passed to dequant");
  if (group_size <= 0 || d % 8 != 0 || d % group_size != 0)
    return fail(B200TP_ERR_UNSUPPORTED_HEAD, "d must be a multiple of 8 and of group_size");
  if ((reinterpret_cast<uintptr_t>(out) & 15) != 0)
    return fail(B200TP_ERR_LOSS_INPUT, "out must be 16-byte aligned");
  return launch_dequant_int4(w_q, scales, biases, qparam_dtype, row0, rows, d, group_size, out, out_dtype,
                             static_cast<cudaStream_t>(stream));
}

}  // extern "C"
