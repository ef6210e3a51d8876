// Host-side helpers: refusal text, device checks, tensor-map construction.
#include "common.h"

#include <cstdlib>
#include <mutex>

namespace b200tp {

static thread_local std::string g_last_error;

void set_last_error(const std::string& msg) { g_last_error = msg; }

int fail(int code, const std::string& msg) {
  g_last_error = msg;
  return code;
}

const char* last_error_cstr() { return g_last_error.c_str(); }

bool pdl_enabled() {
  static const bool on = [] {
    const char* v = getenv("B200TP_NO_PDL");
    return !(v != nullptr && v[0] != '\0' && v[0] != '0');
  }();
  return on;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

int require_sm100() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return fail(B200TP_ERR_NO_DEVICE, "no CUDA device is current");
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess)
    return fail(B200TP_ERR_NO_DEVICE, "cannot query the compute capability");
  if (major != 10)
    return fail(B200TP_ERR_NO_DEVICE,
                "these kernels are built for sm_100a only; the current device is compute capability " +
                    std::to_string(major) + ".x");
  return B200TP_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

static int encode(CUtensorMap* out, CUtensorMapDataType dt, uint32_t rank, const void* base, const cuuint64_t* dims,
                  const cuuint64_t* strides_bytes, const cuuint32_t* box, CUtensorMapSwizzle swz) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return fail(B200TP_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  if ((reinterpret_cast<uintptr_t>(base) & 0xF) != 0)
    return fail(B200TP_ERR_LOSS_INPUT, "tensor base address must be 16-byte aligned for TMA");
  for (uint32_t i = 0; i + 1 < rank; ++i)
    if (strides_bytes[i] % 16 != 0)
      return fail(B200TP_ERR_LOSS_INPUT, "tensor strides must be multiples of 16 bytes for TMA");
  cuuint32_t elem_strides[5] = {1, 1, 1, 1, 1};
  CUresult r = fn(out, dt, rank, const_cast<void*>(base), dims, strides_bytes, box, elem_strides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(B200TP_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult " + std::to_string(static_cast<int>(r)));
  return B200TP_OK;
}

int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride_elems,
                      uint32_t box_rows, uint32_t box_cols) {
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride_elems * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  return encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

int make_tmap_2d_u32(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride_elems,
                     uint32_t box_rows, uint32_t box_cols) {
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride_elems * 4};
  cuuint32_t box[2] = {box_cols, box_rows};
  const CUtensorMapSwizzle swz = box_cols * 4 >= 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  if (box_cols * 4 != 128 && box_cols * 4 != 64)
    return fail(B200TP_ERR_CUDA, "uint32 tensor map: the box must be 64 or 128 bytes wide");
  return encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, base, dims, strides, box, swz);
}

int make_tmap_bhsd_bf16(CUtensorMap* out, const void* base, uint64_t b, uint64_t h, uint64_t s, uint64_t d,
                        int64_t sb, int64_t sh, int64_t ss, uint32_t box_s, uint32_t box_d) {
  cuuint64_t dims[4] = {d, s, h, b};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(ss) * 2, static_cast<cuuint64_t>(sh) * 2,
                           static_cast<cuuint64_t>(sb) * 2};
  cuuint32_t box[4] = {box_d, box_s, 1, 1};
  return encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

int make_tmap_bhsd_f32(CUtensorMap* out, const void* base, uint64_t b, uint64_t h, uint64_t s, uint64_t d,
                       int64_t sb, int64_t sh, int64_t ss, uint32_t box_s, uint32_t box_d) {
  cuuint64_t dims[4] = {d, s, h, b};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(ss) * 4, static_cast<cuuint64_t>(sh) * 4,
                           static_cast<cuuint64_t>(sb) * 4};
  cuuint32_t box[4] = {box_d, box_s, 1, 1};
  return encode(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
}

}  // namespace b200tp
