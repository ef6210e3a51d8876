// Host-side helpers shared by the translation units of the library: refusal bookkeeping,
// CUDA error checks and tiled tensor-map construction through the driver entry point
// (resolved at run time, so the library does not link against libcuda).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <utility>

#include "../../include/b200tp.h"

namespace b200tp {

void set_last_error(const std::string& msg);
int fail(int code, const std::string& msg);

#define B200TP_CUDA_OK(expr)                                                                  \
  do {                                                                                        \
    cudaError_t _e = (expr);                                                                  \
    if (_e != cudaSuccess) {                                                                  \
      return ::b200tp::fail(B200TP_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(_e)); \
    }                                                                                         \
  } while (0)

// Launch with programmatic dependent launch allowed (see ptx.cuh: the kernel must call griddep_wait()).
// The environment variable B200TP_NO_PDL=1 turns the attribute off (plain stream order), for comparisons.
bool pdl_enabled();
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Number of SMs of the current device (cached per device id).
int sm_count();
// 0 when the current device is compute capability 10.x, else a refusal code.
int require_sm100();

// 2-D bf16 tensor map: logical (rows, cols) row-major with `row_stride_elems`, box
// (box_rows, box_cols), 128-byte swizzle, zero fill out of bounds.
int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                      uint64_t row_stride_elems, uint32_t box_rows, uint32_t box_cols);

// 2-D uint32 tensor map (packed 4-bit codes): box (box_rows, box_cols words) of 64 or 128 bytes per row,
// swizzled over that width (64- or 128-byte swizzle), zero fill out of bounds.
int make_tmap_2d_u32(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride_elems,
                     uint32_t box_rows, uint32_t box_cols);

// 4-D bf16 tensor map over (B, H, S, d) with element strides (sb, sh, ss) and unit
// innermost stride: dims (d, S, H, B), box (box_d, box_s, 1, 1), 128-byte swizzle.
int make_tmap_bhsd_bf16(CUtensorMap* out, const void* base, uint64_t b, uint64_t h, uint64_t s, uint64_t d,
                        int64_t sb, int64_t sh, int64_t ss, uint32_t box_s, uint32_t box_d);

// Same but fp32 elements, no swizzle (used by bulk reduce-add of fp32 partials).
int make_tmap_bhsd_f32(CUtensorMap* out, const void* base, uint64_t b, uint64_t h, uint64_t s, uint64_t d,
                       int64_t sb, int64_t sh, int64_t ss, uint32_t box_s, uint32_t box_d);

}  // namespace b200tp
