// Host-side construction of TMA tensor maps.  The driver entry point is resolved through the
// runtime (cudaGetDriverEntryPoint), so the library carries no link-time dependency on libcuda.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tma_host {

typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                    const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                    const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline encode_tiled_fn get_encode_fn() {
  // resolved once per process; the initialisation of a function-local static is thread-safe
  static const encode_tiled_fn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      return reinterpret_cast<encode_tiled_fn>(p);
    }
    return static_cast<encode_tiled_fn>(nullptr);
  }();
  return fn;
}

// A [B, S, H, D] tensor of 16-bit elements with arbitrary (element) strides for B, S, H and unit
// stride for D, tiled as boxes of 64 (D) x 1 (H) x box_rows (S) x 1 (B) with the 128-byte swizzle:
// one box lands in shared memory as `box_rows` rows of 128 bytes.  Out-of-range rows read as zero
// and are dropped on store.  Returns 0 on success.
inline int make_bshd_map(CUtensorMap* map, const void* base, bool is_bf16, int64_t B, int64_t S,
                         int64_t H, int64_t D, int64_t stride_b, int64_t stride_s, int64_t stride_h,
                         uint32_t box_rows) {
  encode_tiled_fn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)S, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)stride_h * 2, (cuuint64_t)stride_s * 2,
                           (cuuint64_t)stride_b * 2};
  cuuint32_t box[4] = {64, 1, box_rows, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                  4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

// A 4-D f32 tensor (innermost stride 1; `strides` in BYTES for dimensions 1..3, multiples of 16)
// tiled with the 128-byte swizzle: box[0] must be 32 elements (128 bytes).  Out-of-range elements
// read as zero.  Returns 0 on success.
inline int make_f32_map_sw128(CUtensorMap* map, const void* base, const uint64_t dims[4],
                              const uint64_t strides[3], const uint32_t box[4]) {
  encode_tiled_fn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t d[4] = {dims[0], dims[1], dims[2], dims[3]};
  cuuint64_t st[3] = {strides[0], strides[1], strides[2]};
  cuuint32_t bx[4] = {box[0], box[1], box[2], box[3]};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(base), d, st, bx, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

}  // namespace tma_host
