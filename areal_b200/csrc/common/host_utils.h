// Host-side helpers shared by the kernel launchers: TMA tensor-map encoding
// through the driver entry point (no link-time dependency on libcuda), the
// per-process error word that kernels write when a bounded wait gives up, and
// a uniform way of returning CUDA errors through the C ABI.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

namespace b200 {

// All exported launchers return 0 on success, a negative cudaError_t otherwise.
#define B200_CHECK(expr)                                                          \
  do {                                                                            \
    cudaError_t _e = (expr);                                                      \
    if (_e != cudaSuccess) {                                                      \
      fprintf(stderr, "[areal_b200] %s failed at %s:%d: %s\n", #expr, __FILE__,   \
              __LINE__, cudaGetErrorString(_e));                                  \
      return -static_cast<int>(_e);                                               \
    }                                                                             \
  } while (0)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) !=
            cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      return nullptr;
    }
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D row-major tensor [rows, cols] of `elem_bytes`-wide elements with row
// pitch `row_stride_bytes`; box = [box_rows, box_cols]; 128-byte swizzle when
// box_cols * elem_bytes == 128, none otherwise. Out-of-range reads fill zero.
inline int make_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dt,
                        uint32_t elem_bytes, uint64_t rows, uint64_t cols,
                        uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_cols,
                        bool swizzle128 = true) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr,
            "[areal_b200] cuTensorMapEncodeTiled failed (%d): base=%p rows=%llu cols=%llu "
            "stride=%llu box=[%u,%u]\n",
            (int)r, base, (unsigned long long)rows, (unsigned long long)cols,
            (unsigned long long)row_stride_bytes, box_rows, box_cols);
    return -2;
  }
  return 0;
}

// 3-D variant: [depth, rows, cols], strides in bytes for rows and depth.
inline int make_tmap_3d(CUtensorMap* out, const void* base, CUtensorMapDataType dt,
                        uint64_t depth, uint64_t rows, uint64_t cols, uint64_t row_stride_bytes,
                        uint64_t depth_stride_bytes, uint32_t box_rows, uint32_t box_cols,
                        bool swizzle128 = true) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t gdim[3] = {cols, rows, depth};
  cuuint64_t gstride[2] = {row_stride_bytes, depth_stride_bytes};
  cuuint32_t box[3] = {box_cols, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, dt, 3, const_cast<void*>(base), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "[areal_b200] cuTensorMapEncodeTiled(3d) failed (%d)\n", (int)r);
    return -2;
  }
  return 0;
}

// Device status word shared by all launches of this process on the current
// device. Kernels atomically set it to a non-zero code when a bounded wait
// expires; the host reads it with b200_read_status().
int* device_status_word();

inline int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

}  // namespace b200
