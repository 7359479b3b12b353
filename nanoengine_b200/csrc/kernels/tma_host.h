// Host side of TMA: build CUtensorMap descriptors for row-major 2-D / 3-D tensors.  The driver entry point
// is looked up at run time, so the library links against cudart only and loads on machines without a driver.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

namespace ne {

enum TmaDtype : int { TMA_U8 = 0, TMA_BF16 = 1, TMA_F32 = 2 };
enum TmaSwizzle : int { TMA_SW_NONE = 0, TMA_SW_32 = 1, TMA_SW_64 = 2, TMA_SW_128 = 3 };

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) return nullptr;
    fn = (EncodeTiledFn)p;
  }
  return fn;
}

// dims/box are innermost first.  strides_bytes has rank-1 entries (stride of dim 1, dim 2, ...).
// Returns 0 on success.  Base must be 16-byte aligned and every stride a multiple of 16 bytes.
inline int make_tmap(CUtensorMap* out, const void* base, int dtype, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                     const uint32_t* box, int swizzle) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return -1;
  if (((uintptr_t)base & 15) != 0) return -2;
  CUtensorMapDataType dt = dtype == TMA_U8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : dtype == TMA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUtensorMapSwizzle sw = swizzle == TMA_SW_128 ? CU_TENSOR_MAP_SWIZZLE_128B : swizzle == TMA_SW_64 ? CU_TENSOR_MAP_SWIZZLE_64B
                          : swizzle == TMA_SW_32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE;
  cuuint64_t d[5]; cuuint64_t s[5]; cuuint32_t b[5]; cuuint32_t e[5];
  for (int i = 0; i < rank; i++) { d[i] = dims[i]; b[i] = box[i]; e[i] = 1; }
  for (int i = 0; i + 1 < rank; i++) { s[i] = strides_bytes[i]; if (s[i] & 15) return -3; }
  CUresult r = fn(out, dt, (cuuint32_t)rank, const_cast<void*>(base), d, s, b, e, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { fprintf(stderr, "ne: cuTensorMapEncodeTiled failed (%d)\n", (int)r); return (int)r; }
  return 0;
}

}  // namespace ne
