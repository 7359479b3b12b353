// NVFP4 activation quantiser: bf16 rows -> packed e2m1 (two per byte, low nibble first) + one UE4M3 scale per 16 elements.
//
// Recipe (the one ModelOpt NVFP4 checkpoints assume for their `input_scale`): with g = 1 / input_scale,
//   sf = e4m3(g * amax16 / 6),   q = e2m1(x * g / sf)        so that   x ~= q * sf * input_scale,
// and the GEMM multiplies its accumulator by alpha = input_scale * weight_scale_2.  `g` is one number for the whole matrix or one
// per expert of the contiguous grouped layout (rows [row_start[e], row_start[e] + counts[e]) belong to expert e; rows outside
// every expert's range are skipped).
//
// Replaces in the reference: flashinfer `fp4_quantize` / `scaled_fp4_grouped_quantize` /
// `silu_and_mul_scaled_nvfp4_experts_quantize` as called from kernel/cutedsl_nvfp4_moe.py and layers/backends/experts/nvfp4.py:318-326.
#include <cuda_fp4.h>

#include "ptx.cuh"

namespace ne {

// one thread per 16 elements
__global__ void __launch_bounds__(256) nvfp4_quant_kernel(const __nv_bfloat16* __restrict__ x, long long x_ld, uint8_t* __restrict__ q,
                                                          uint8_t* __restrict__ sf, const float* __restrict__ gscale, const int* __restrict__ row_start,
                                                          const int* __restrict__ counts, int groups, int R, int K) {
  pdl_wait(); pdl_trigger();
  const int per_row = K / 16;
  const long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (item >= (long long)R * per_row) return;
  const int row = (int)(item / per_row), c = (int)(item % per_row);
  float g = gscale[0];
  if (row_start) {
    // the expert whose range holds this row: the last one that starts at or before it
    int lo = 0, hi = groups - 1;
    while (lo < hi) { const int mid = (lo + hi + 1) >> 1; if (row_start[mid] <= row) lo = mid; else hi = mid - 1; }
    if (row < row_start[lo] || row >= row_start[lo] + counts[lo]) return;
    g = gscale[lo];
  }
  const uint4* src = reinterpret_cast<const uint4*>(x + (long long)row * x_ld + c * 16);
  const uint4 v0 = src[0], v1 = src[1];
  const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
  float f[16];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const float2 p = unpack_bf16x2(w[i]);
    f[2 * i] = p.x; f[2 * i + 1] = p.y;
    amax = fmaxf(amax, fmaxf(fabsf(p.x), fabsf(p.y)));
  }
  const uint8_t sfb = to_e4m3(g * amax * (1.f / 6.f));
  const float sfv = e4m3_to_float(sfb);
  const float os = sfv != 0.f ? g / sfv : 0.f;
  uint32_t out[2] = {0u, 0u};
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const uint32_t b = (uint32_t)__nv_cvt_float2_to_fp4x2(make_float2(f[2 * i] * os, f[2 * i + 1] * os), __NV_E2M1, cudaRoundNearest);
    out[i >> 2] |= (b & 0xffu) << (8 * (i & 3));
  }
  *reinterpret_cast<uint2*>(q + (long long)row * (K / 2) + c * 8) = make_uint2(out[0], out[1]);
  sf[(long long)row * per_row + c] = sfb;
}

}  // namespace ne

using namespace ne;

extern "C" int ne_nvfp4_quant(const void* x, long long x_ld, void* q, void* sf, const float* gscale, const int* row_start, const int* counts,
                              int groups, int R, int K, cudaStream_t st) {
  if (R <= 0) return 0;
  if (K % 16 != 0 || x_ld % 8 != 0 || (row_start && (!counts || groups < 1))) return 1001;
  const long long items = (long long)R * (K / 16);
  return (int)launch_pdl(nvfp4_quant_kernel, dim3((unsigned)((items + 255) / 256)), dim3(256), 0, st, (const __nv_bfloat16*)x, x_ld, (uint8_t*)q,
                         (uint8_t*)sf, gscale, row_start, counts, groups, R, K);
}
