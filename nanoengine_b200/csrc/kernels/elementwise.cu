// Memory-bound operators of the decoder layer, each fused as far as its neighbours allow:
//   * (residual add +) RMSNorm (+ 1x128 fp8 quantisation with the scale layout the block-scaled GEMM reads)
//   * 1x128 fp8 quantisation of bf16 activations
//   * SwiGLU (+ 1x128 fp8 requantisation), flat or over the masked [E, max_m, *] expert layout
//   * RoPE in place on a strided sub-range of each head (MLA q_pe / k_pe, GQA q / k)
//   * MLA latent KV row store into the paged cache (bf16 rows or raw 576-byte e4m3 rows)
// Replaces in the reference: triton/generic/rmsnorm.py, triton/hopper/rmsnorm_quant_fp8.py:27-108, triton/hopper/fp8.py:9-187,
// jit/sgl/csrc/deepseek_v4/silu_and_mul_masked_post_quant.cuh, triton/hopper/mla_rope.py:17, triton/generic/kv_store.py,
// triton/hopper/fp8_utils.py:203-305.
#include "ptx.cuh"

namespace ne {

constexpr float kFp8Max = 448.f;

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < nw) ? red[threadIdx.x] : 0.f;
  if (w == 0) { t = warp_sum(t); if (l == 0) red[0] = t; }
  __syncthreads();
  float r = red[0];
  __syncthreads();
  return r;
}

// One CTA per row.  x may be a strided view (row stride x_ld).  Optional residual add (res_in -> res_out, bf16),
// optional bf16 output, optional fp8 output with scales written to sc[(col/128) * sc_ld + row].
__global__ void __launch_bounds__(256) rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, long long x_ld, const __nv_bfloat16* __restrict__ res_in,
                                                     const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out, long long out_ld,
                                                     __nv_bfloat16* __restrict__ res_out, uint8_t* __restrict__ q, float* __restrict__ sc, int sc_ld,
                                                     int H, float eps, float w_off, int pow2) {
  pdl_wait(); pdl_trigger();      // dependent launch: nothing above this line touches global memory
  extern __shared__ float srow[];            // H floats
  __shared__ float red[32];
  const int row = blockIdx.x;
  const __nv_bfloat16* xr = x + (long long)row * x_ld;
  float ss = 0.f;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    uint4 v = *reinterpret_cast<const uint4*>(xr + i);
    uint32_t u[4] = {v.x, v.y, v.z, v.w};
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; j++) { float2 t = unpack_bf16x2(u[j]); f[2 * j] = t.x; f[2 * j + 1] = t.y; }
    if (res_in) {
      uint4 rv = *reinterpret_cast<const uint4*>(res_in + (long long)row * H + i);
      uint32_t ru[4] = {rv.x, rv.y, rv.z, rv.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        float2 t = unpack_bf16x2(ru[j]);
        o[j] = pack_bf16x2(f[2 * j] + t.x, f[2 * j + 1] + t.y);
        float2 b = unpack_bf16x2(o[j]);      // the sum is rounded to bf16 first, as the unfused form does
        f[2 * j] = b.x; f[2 * j + 1] = b.y;
      }
      *reinterpret_cast<uint4*>(res_out + (long long)row * H + i) = make_uint4(o[0], o[1], o[2], o[3]);
    } else if (res_out) {
      *reinterpret_cast<uint4*>(res_out + (long long)row * H + i) = v;
    }
#pragma unroll
    for (int j = 0; j < 8; j++) { srow[i + j] = f[j]; ss += f[j] * f[j]; }
  }
  float tot = block_sum(ss, red);
  float inv = rsqrtf(tot / (float)H + eps);
  if (out) {
    for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
      uint4 wv = *reinterpret_cast<const uint4*>(w + i);
      uint32_t wu[4] = {wv.x, wv.y, wv.z, wv.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        float2 t = unpack_bf16x2(wu[j]);
        o[j] = pack_bf16x2(srow[i + 2 * j] * inv * (t.x + w_off), srow[i + 2 * j + 1] * inv * (t.y + w_off));
      }
      *reinterpret_cast<uint4*>(out + (long long)row * out_ld + i) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
  if (q) {
    // one warp per 128-column group; values are rounded to bf16 first so the result matches quantising the bf16 output
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int g = warp; g < H / 128; g += nw) {
      int c = g * 128 + lane * 4;
      float v[4];
      float amax = 0.f;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        v[j] = __bfloat162float(__float2bfloat16(srow[c + j] * inv * (__bfloat162float(w[c + j]) + w_off)));
        amax = fmaxf(amax, fabsf(v[j]));
      }
      amax = fmaxf(warp_max(amax), 1e-10f);
      float is; const float s = fp8_group_scale(amax, pow2, &is);
      *reinterpret_cast<uint32_t*>(q + (long long)row * H + c) = pack_e4m3x4(v[0] * is, v[1] * is, v[2] * is, v[3] * is);
      if (lane == 0) sc[(long long)g * sc_ld + row] = s;
    }
  }
}

// bf16 [T, K] (row stride x_ld) -> e4m3 [T, K] + scales sc[(k/128) * sc_ld + t].  One warp per (row, group).
__global__ void quant_1x128_kernel(const __nv_bfloat16* __restrict__ x, long long x_ld, uint8_t* __restrict__ q, float* __restrict__ sc,
                                   int sc_ld, int T, int K, int pow2) {
  pdl_wait(); pdl_trigger();      // dependent launch: nothing above this line touches global memory
  const int groups = K / 128;
  long long gw = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (gw >= (long long)T * groups) return;
  int row = (int)(gw / groups), g = (int)(gw % groups), lane = threadIdx.x & 31;
  uint2 v = *reinterpret_cast<const uint2*>(x + (long long)row * x_ld + g * 128 + lane * 4);
  float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y);
  float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
  amax = fmaxf(warp_max(amax), 1e-10f);
  float is; const float s = fp8_group_scale(amax, pow2, &is);
  *reinterpret_cast<uint32_t*>(q + (long long)row * K + g * 128 + lane * 4) = pack_e4m3x4(a.x * is, a.y * is, b.x * is, b.y * is);
  if (lane == 0) sc[(long long)g * sc_ld + row] = s;
}

__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }

// One (row, 128-column block) item of SwiGLU: 4 columns per lane; bf16 out, or e4m3 with the block's scale at sc[c * sc_ld + row].
// Gated activation of one (gate, up) pair.  act 0: silu(g) u.  act 1 (clamped SwiGLU, limit p0): up in [-p0, p0], gate <= p0,
// then silu(g) u (reference layers/activation.py:86-92).  act 2 (SiTU-GLU, p0 = beta, p1 = linear beta or 0):
// beta tanh(g / beta) sigmoid(g) times p1 tanh(u / p1) (reference kernel/triton/generic/situ.py:24-27).  act 3: GELU(g) u with the
// tanh approximation (reference models/gemma4/gemma4.py:27-36).
__device__ __forceinline__ float glu_act(float g, float u, int act, float p0, float p1) {
  if (act == 3) return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * u;      // tanh-approximated GELU
  if (act == 1) { u = fminf(fmaxf(u, -p0), p0); g = fminf(g, p0); }
  else if (act == 2) {
    if (p1 > 0.f) u = p1 * tanhf(u / p1);
    return p0 * tanhf(g / p0) / (1.f + __expf(-g)) * u;
  }
  return silu(g) * u;
}

__device__ __forceinline__ void silu_item(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, uint8_t* __restrict__ q,
                                          float* __restrict__ sc, int sc_ld, long long mrow, int row, int c, int I, int lane,
                                          int act, float p0, float p1, int pow2) {
  const __nv_bfloat16* xr = x + mrow * 2 * I + c * 128 + lane * 4;
  uint2 gv = *reinterpret_cast<const uint2*>(xr), uv = *reinterpret_cast<const uint2*>(xr + I);
  float2 g0 = unpack_bf16x2(gv.x), g1 = unpack_bf16x2(gv.y), u0 = unpack_bf16x2(uv.x), u1 = unpack_bf16x2(uv.y);
  float v[4] = {glu_act(g0.x, u0.x, act, p0, p1), glu_act(g0.y, u0.y, act, p0, p1), glu_act(g1.x, u1.x, act, p0, p1), glu_act(g1.y, u1.y, act, p0, p1)};
  const long long o = mrow * I + c * 128 + lane * 4;
  if (!q) {
    *reinterpret_cast<uint2*>(y + o) = make_uint2(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]));
    return;
  }
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 4; j++) { v[j] = __bfloat162float(__float2bfloat16(v[j])); amax = fmaxf(amax, fabsf(v[j])); }
  amax = fmaxf(warp_max(amax), 1e-10f);
  float is; const float s = fp8_group_scale(amax, pow2, &is);
  *reinterpret_cast<uint32_t*>(q + o) = pack_e4m3x4(v[0] * is, v[1] * is, v[2] * is, v[3] * is);
  if (lane == 0) sc[(long long)c * sc_ld + row] = s;
}

// x [groups, rows, 2I] -> y.  One warp per (row, 128 output columns).  rows_valid[g] masks rows (nullptr = all).
// Output bf16 (q == nullptr) or e4m3 + scales sc[g][(col/128) * sc_ld + row].
constexpr int kSiluMaxGroups = 1024;
__global__ void silu_mul_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, uint8_t* __restrict__ q, float* __restrict__ sc,
                                int sc_ld, long long sc_gs, const int* __restrict__ rows_valid, const int* __restrict__ row_start, int groups,
                                int rows, int I, int act, float p0, float p1, int pow2) {
  pdl_wait(); pdl_trigger();      // dependent launch: nothing above this line touches global memory
  // warps stride over the concatenation of all groups' (valid row, 128-column block) items, so a sparsely filled masked
  // layout costs only its valid rows and every warp gets an equal share whatever the split between groups.  The item index
  // is mapped back to its group through a table of first-item indices built once per CTA in shared memory and a binary
  // search: walking the groups in every warp (with a global load and 64-bit modulo arithmetic per group) made a kernel
  // that moves 10 MB take 30 us.
  __shared__ int s_first[kSiluMaxGroups + 1], s_rs[kSiluMaxGroups];
  const int cg = I / 128, lane = threadIdx.x & 31;
  if (groups <= kSiluMaxGroups) {
    for (int g = threadIdx.x; g < groups; g += blockDim.x) {
      int n = rows_valid ? rows_valid[g] : rows;
      n = n < rows ? n : rows;
      s_first[g + 1] = (n > 0 ? n : 0) * cg;
      s_rs[g] = row_start ? row_start[g] : 0;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
      const int per = (groups + 31) / 32, lo = lane * per, hi = lo + per < groups ? lo + per : groups;
      int sum = 0;
      for (int i = lo; i < hi; i++) sum += s_first[i + 1];
      int incl = sum;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) { const int v = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += v; }
      int run = incl - sum;
      if (lane == 0) s_first[0] = 0;
      for (int i = lo; i < hi; i++) { run += s_first[i + 1]; s_first[i + 1] = run; }
    }
    __syncthreads();
    const int total = s_first[groups];
    const int w0 = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), nw = gridDim.x * (blockDim.x >> 5);
    int g = 0;
    for (int it = w0; it < total; it += nw) {
      int hi = groups - 1;                              // items only move forward: search from the last group found
      while (g < hi) { const int mid = (g + hi + 1) >> 1; if (s_first[mid] <= it) g = mid; else hi = mid - 1; }
      const int l = it - s_first[g];
      const int ri = l / cg, c = l - ri * cg;
      const int row = s_rs[g] + ri;
      if (row >= rows && row_start) continue;
      const long long gbase = row_start ? 0 : (long long)g * rows;
      silu_item(x, y, q, sc + (row_start ? 0 : (long long)g * sc_gs), sc_ld, gbase + row, row, c, I, lane, act, p0, p1, pow2);
    }
    return;
  }
  // more groups than the table holds: walk them
  const long long w0 = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nw = (long long)gridDim.x * (blockDim.x >> 5);
  long long base = 0;                      // items of the groups before g, modulo nw
  for (int g = 0; g < groups; g++) {
    int nrows = rows_valid ? rows_valid[g] : rows;
    nrows = nrows < rows ? nrows : rows;
    const long long gbase = row_start ? 0 : (long long)g * rows;
    const int r0 = row_start ? row_start[g] : 0;
    const long long items = (long long)nrows * cg;
    long long first = w0 - base;
    if (first < 0) first += nw;
    base = (base + items) % nw;
    for (long long it = first; it < items; it += nw) {
      const int row = r0 + (int)(it / cg), c = (int)(it % cg);
      if (row >= rows && row_start) continue;
      silu_item(x, y, q, sc + (row_start ? 0 : (long long)g * sc_gs), sc_ld, gbase + row, row, c, I, lane, act, p0, p1, pow2);
    }
  }
}

// Rotary embedding on dims [off, off+D) of each of `heads` heads of every row; the result goes to `y` (which may be `x`
// itself for the in-place form, or a differently strided buffer such as the rope tail of the absorbed-query tensor).
// cache [max_pos, D] fp32 (cos | sin).  interleaved: pairs (2i, 2i+1); otherwise pairs (i, i + D/2).
__global__ void rope_kernel(const __nv_bfloat16* __restrict__ x, long long row_stride, int head_stride, __nv_bfloat16* __restrict__ y,
                            long long y_row_stride, int y_head_stride, int heads, int off, int D,
                            const long long* __restrict__ positions, const float* __restrict__ cache, int interleaved, int T) {
  pdl_wait(); pdl_trigger();      // dependent launch: nothing above this line touches global memory
  int half = D / 2;
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long total = (long long)T * heads * half;
  if (idx >= total) return;
  int i = (int)(idx % half); long long r = idx / half; int h = (int)(r % heads); int t = (int)(r / heads);
  const float* cs = cache + positions[t] * D;
  float c = cs[i], s = cs[half + i];
  const __nv_bfloat16* p = x + (long long)t * row_stride + (long long)h * head_stride + off;
  __nv_bfloat16* q = y + (long long)t * y_row_stride + (long long)h * y_head_stride;
  int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + half;
  float a = __bfloat162float(p[ia]), b = __bfloat162float(p[ib]);
  q[ia] = __float2bfloat16(a * c - b * s);
  q[ib] = __float2bfloat16(b * c + a * s);
}

// MLA key path in one pass, one warp per token: RMSNorm of the compressed KV (R values, rounded to bf16 as the separate
// norm kernel would), interleaved RoPE of the R..R+rope tail, and the store of both into the token's cache row (bf16, or
// e4m3 with a clamped cast and no scale).  kv [T, >= R + rope] bf16 with row stride kv_ld.
__global__ void __launch_bounds__(256) mla_kv_prepare_kernel(const __nv_bfloat16* __restrict__ kv, long long kv_ld, const __nv_bfloat16* __restrict__ w,
                                                            float eps, const long long* __restrict__ positions, const float* __restrict__ rope_cache,
                                                            void* __restrict__ cache, const long long* __restrict__ slots, int T, int R, int rope, int fp8) {
  pdl_wait(); pdl_trigger();      // dependent launch: nothing above this line touches global memory
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= T) return;
  const long long slot = slots[t];
  if (slot >= 0 && !NE_INDEX_OK(slot, BK_CACHE_ROWS, 20, __LINE__)) return;
  const __nv_bfloat16* row = kv + (long long)t * kv_ld;
  float ss = 0.f;
  for (int c = lane * 2; c < R; c += 64) {
    const float2 f = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(row + c));
    ss += f.x * f.x + f.y * f.y;
  }
  ss = warp_sum(ss);
  if (slot < 0) return;
  const float inv = rsqrtf(ss / (float)R + eps);
  const int D = R + rope;
  for (int c = lane * 2; c < R; c += 64) {
    const float2 f = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(row + c));
    const float2 g = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(w + c));
    const uint32_t o = pack_bf16x2(f.x * inv * g.x, f.y * inv * g.y);
    if (fp8) {
      const float2 r = unpack_bf16x2(o);
      *reinterpret_cast<uint16_t*>(reinterpret_cast<uint8_t*>(cache) + slot * D + c) = (uint16_t)__nv_cvt_float2_to_fp8x2(r, __NV_SATFINITE, __NV_E4M3);
    } else {
      *reinterpret_cast<uint32_t*>(reinterpret_cast<__nv_bfloat16*>(cache) + slot * D + c) = o;
    }
  }
  const float* cs = rope_cache + positions[t] * rope;
  const int half = rope / 2;
  for (int i = lane; i < half; i += 32) {
    const float2 f = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(row + R + 2 * i));
    const float c = cs[i], sn = cs[half + i];
    const uint32_t o = pack_bf16x2(f.x * c - f.y * sn, f.y * c + f.x * sn);
    if (fp8) {
      const float2 r = unpack_bf16x2(o);
      *reinterpret_cast<uint16_t*>(reinterpret_cast<uint8_t*>(cache) + slot * D + R + 2 * i) = (uint16_t)__nv_cvt_float2_to_fp8x2(r, __NV_SATFINITE, __NV_E4M3);
    } else {
      *reinterpret_cast<uint32_t*>(reinterpret_cast<__nv_bfloat16*>(cache) + slot * D + R + 2 * i) = o;
    }
  }
}

// Absorbed MLA query for the fp8 attention kernel: q8[t, h, :] = e4m3([q_lat[t, h, :R] | rope(q_pe[t, h, :])]) with a
// clamped cast and no scale; q_pe is the interleaved rope tail of the query projection (a strided view).  One warp per
// (token, head).
__global__ void __launch_bounds__(256) mla_q_finalize_kernel(const __nv_bfloat16* __restrict__ q_lat, const __nv_bfloat16* __restrict__ q_pe,
                                                            long long pe_row_stride, int pe_head_stride, const long long* __restrict__ positions,
                                                            const float* __restrict__ rope_cache, uint8_t* __restrict__ q8, int T, int H, int R, int rope) {
  pdl_wait(); pdl_trigger();      // dependent launch: nothing above this line touches global memory
  const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (wid >= (long long)T * H) return;
  const int t = (int)(wid / H), h = (int)(wid % H);
  const int D = R + rope;
  const __nv_bfloat16* src = q_lat + wid * R;
  uint8_t* dst = q8 + wid * D;
  for (int c = lane * 8; q_lat && c < R; c += 256) {        // q_lat == nullptr: the producing GEMM already wrote the e4m3 latent part
    const uint4 v = *reinterpret_cast<const uint4*>(src + c);
    const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c2 = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
    *reinterpret_cast<uint2*>(dst + c) = make_uint2(pack_e4m3x4(a.x, a.y, b.x, b.y), pack_e4m3x4(c2.x, c2.y, d.x, d.y));
  }
  const float* cs = rope_cache + positions[t] * rope;
  const int half = rope / 2;
  const __nv_bfloat16* pe = q_pe + (long long)t * pe_row_stride + (long long)h * pe_head_stride;
  for (int i = lane; i < half; i += 32) {
    const float2 f = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(pe + 2 * i));
    const float c = cs[i], sn = cs[half + i];
    const float2 r = unpack_bf16x2(pack_bf16x2(f.x * c - f.y * sn, f.y * c + f.x * sn));     // bf16 rounding as the unfused rope
    *reinterpret_cast<uint16_t*>(dst + R + 2 * i) = (uint16_t)__nv_cvt_float2_to_fp8x2(r, __NV_SATFINITE, __NV_E4M3);
  }
}

// cache row = [ckv (R) | k_pe (rope)], bf16 or e4m3 (clamped cast, no scale).  One warp per token.
__global__ void mla_kv_store_kernel(const __nv_bfloat16* __restrict__ ckv, long long ckv_ld, const __nv_bfloat16* __restrict__ kpe, long long kpe_ld,
                                    void* __restrict__ cache, const long long* __restrict__ slots, int T, int R, int rope, int fp8) {
  int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= T) return;
  long long slot = slots[t];
  if (slot >= 0 && !NE_INDEX_OK(slot, BK_CACHE_ROWS, 20, __LINE__)) return;
  if (slot < 0) return;
  int D = R + rope;
  for (int c = lane * 2; c < D; c += 64) {
    uint32_t v = c < R ? *reinterpret_cast<const uint32_t*>(ckv + (long long)t * ckv_ld + c)
                       : *reinterpret_cast<const uint32_t*>(kpe + (long long)t * kpe_ld + (c - R));
    if (fp8) {
      float2 f = unpack_bf16x2(v);
      uint16_t o = (uint16_t)__nv_cvt_float2_to_fp8x2(f, __NV_SATFINITE, __NV_E4M3);
      *reinterpret_cast<uint16_t*>(reinterpret_cast<uint8_t*>(cache) + slot * D + c) = o;
    } else {
      *reinterpret_cast<uint32_t*>(reinterpret_cast<__nv_bfloat16*>(cache) + slot * D + c) = v;
    }
  }
}

// y[t, :] = a[t, :] + b[t, :] (bf16), used where a fused epilogue is not available
__global__ void add_kernel(const __nv_bfloat16* a, const __nv_bfloat16* b, __nv_bfloat16* y, long long n) {
  pdl_wait(); pdl_trigger();      // dependent launch: nothing above this line touches global memory
  long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= n) return;
  uint4 av = *reinterpret_cast<const uint4*>(a + i), bv = *reinterpret_cast<const uint4*>(b + i);
  uint32_t au[4] = {av.x, av.y, av.z, av.w}, bu[4] = {bv.x, bv.y, bv.z, bv.w}, o[4];
#pragma unroll
  for (int j = 0; j < 4; j++) { float2 p = unpack_bf16x2(au[j]), r = unpack_bf16x2(bu[j]); o[j] = pack_bf16x2(p.x + r.x, p.y + r.y); }
  *reinterpret_cast<uint4*>(y + i) = make_uint4(o[0], o[1], o[2], o[3]);
}


// GQA front end in one pass over the qkv projection output: per-head RMSNorm of q and k (optional), rotary embedding of both
// (pairs (i, i + D/2), the whole head rotated) and the store of k and v into their paged cache rows.  One warp per (token, head);
// a lane owns the bf16 pairs at columns 2*lane + 64*j, so with D = 128 or 256 both halves of every rotation pair sit in the
// same lane.  qkv [T, (Hq + 2*Hkv) * D] with row stride ld; q_out [T, Hq, D] contiguous; caches [slots, Hkv, D].
// Replaces four launches (q norm, k norm, two rope passes) and an indexed copy.  Reference: triton/generic/kv_store.py:7,31,
// kernel/jit/sgl/csrc/deepseek_v4/fused_norm_rope.cuh:42, models/qwen3_moe/qwen3_moe.py:58-146.
template <int D>
__global__ void __launch_bounds__(256) gqa_qkv_prepare_kernel(const __nv_bfloat16* __restrict__ qkv, long long ld, int Hq, int Hkv,
                                                             const __nv_bfloat16* __restrict__ qw, const __nv_bfloat16* __restrict__ kw, float eps,
                                                             float w_offset, const long long* __restrict__ positions,
                                                             const float* __restrict__ rope_cache, __nv_bfloat16* __restrict__ q_out,
                                                             __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                                             const long long* __restrict__ slots, int T) {
  pdl_wait(); pdl_trigger();
  constexpr int J = D / 64;                       // bf16 pairs per lane
  const int heads = Hq + 2 * Hkv;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (long long)T * heads) return;
  const int t = (int)(w / heads), h = (int)(w - (long long)t * heads), lane = threadIdx.x & 31;
  const __nv_bfloat16* src = qkv + (long long)t * ld + (long long)h * D;
  float2 v[J];
#pragma unroll
  for (int j = 0; j < J; j++) v[j] = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(src + 2 * lane + 64 * j));
  const bool is_q = h < Hq, is_k = !is_q && h < Hq + Hkv;
  const long long slot = is_q ? 0 : slots[t];
  if (slot >= 0 && !NE_INDEX_OK(slot, BK_CACHE_ROWS, 20, __LINE__)) return;
  if (!is_q && slot < 0) return;                  // padded token: nothing to store
  if (is_q || is_k) {
    const __nv_bfloat16* nw = is_q ? qw : kw;
    if (nw) {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < J; j++) ss += v[j].x * v[j].x + v[j].y * v[j].y;
      const float r = rsqrtf(warp_sum(ss) / D + eps);
#pragma unroll
      for (int j = 0; j < J; j++) {
        const float2 g = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(nw + 2 * lane + 64 * j));
        // the separate norm kernel rounds to bf16 before the rotation reads it: keep that rounding
        v[j] = unpack_bf16x2(pack_bf16x2(v[j].x * r * (g.x + w_offset), v[j].y * r * (g.y + w_offset)));
      }
    }
    const float* cs = rope_cache + positions[t] * D;      // [cos (D/2) | sin (D/2)]
#pragma unroll
    for (int j = 0; j < J / 2; j++) {
      const int i = 2 * lane + 64 * j;                    // column of the first element of the pair's low half
      const float2 c = *reinterpret_cast<const float2*>(cs + i), sn = *reinterpret_cast<const float2*>(cs + D / 2 + i);
      const float2 a = v[j], b = v[j + J / 2];
      v[j] = make_float2(a.x * c.x - b.x * sn.x, a.y * c.y - b.y * sn.y);
      v[j + J / 2] = make_float2(b.x * c.x + a.x * sn.x, b.y * c.y + a.y * sn.y);
    }
  }
  __nv_bfloat16* dst = is_q ? q_out + ((long long)t * Hq + h) * D
                            : (is_k ? k_cache + (slot * Hkv + (h - Hq)) * D : v_cache + (slot * Hkv + (h - Hq - Hkv)) * D);
#pragma unroll
  for (int j = 0; j < J; j++) *reinterpret_cast<uint32_t*>(dst + 2 * lane + 64 * j) = pack_bf16x2(v[j].x, v[j].y);
}

// Stand-alone paged store of K and V rows ([T, Hkv, D] each, any row stride) for shapes the fused front end does not take.
__global__ void __launch_bounds__(256) gqa_kv_store_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v, long long k_ld,
                                                          long long v_ld, __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                                          const long long* __restrict__ slots, int T, int row_elems) {
  pdl_wait(); pdl_trigger();
  const int t = blockIdx.x;
  const long long slot = slots[t];
  if (slot >= 0 && !NE_INDEX_OK(slot, BK_CACHE_ROWS, 20, __LINE__)) return;
  if (slot < 0) return;
  for (int c = threadIdx.x * 8; c < row_elems; c += blockDim.x * 8) {
    *reinterpret_cast<uint4*>(k_cache + slot * row_elems + c) = *reinterpret_cast<const uint4*>(k + (long long)t * k_ld + c);
    *reinterpret_cast<uint4*>(v_cache + slot * row_elems + c) = *reinterpret_cast<const uint4*>(v + (long long)t * v_ld + c);
  }
}

// GELU over a flat bf16 array, 8 elements per thread: tanh approximation or the exact erf form
__global__ void __launch_bounds__(256) gelu_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n, int tanh_form) {
  pdl_wait(); pdl_trigger();
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= n) return;
  auto act = [&](float v) {
    return tanh_form ? 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v))) : 0.5f * v * (1.f + erff(v * 0.7071067811865476f));
  };
  if (i + 8 <= n) {
    const uint4 u = *reinterpret_cast<const uint4*>(x + i);
    float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
    *reinterpret_cast<uint4*>(y + i) = make_uint4(pack_bf16x2(act(a.x), act(a.y)), pack_bf16x2(act(b.x), act(b.y)), pack_bf16x2(act(c.x), act(c.y)),
                                                  pack_bf16x2(act(d.x), act(d.y)));
  } else {
    for (long long j = i; j < n; j++) y[j] = __float2bfloat16(act(__bfloat162float(x[j])));
  }
}

// LayerNorm over the last dimension, one warp per row: y = (x - mean) / sqrt(var + eps) * w + b.
__global__ void __launch_bounds__(256) layernorm_kernel(const __nv_bfloat16* __restrict__ x, long long ld, const __nv_bfloat16* __restrict__ w,
                                                       const __nv_bfloat16* __restrict__ b, float eps, __nv_bfloat16* __restrict__ y, long long rows, int D) {
  pdl_wait(); pdl_trigger();
  const long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const int lane = threadIdx.x & 31;
  const __nv_bfloat16* xr = x + r * ld;
  float s = 0.f, ss = 0.f;
  for (int c = lane; c < D; c += 32) { const float f = __bfloat162float(xr[c]); s += f; ss += f * f; }
  s = warp_sum(s); ss = warp_sum(ss);
  const float mean = s / D, rstd = rsqrtf(fmaxf(ss / D - mean * mean, 0.f) + eps);
  for (int c = lane; c < D; c += 32) {
    const float f = (__bfloat162float(xr[c]) - mean) * rstd;
    y[r * D + c] = __float2bfloat16(f * (w ? __bfloat162float(w[c]) : 1.f) + (b ? __bfloat162float(b[c]) : 0.f));
  }
}

// Merge of two attention partials by their log-sum-exp: o = (e^{l1} o1 + e^{l2} o2) / (e^{l1} + e^{l2}), lse = log(e^{l1} + e^{l2}).
// o1, o2, out [rows, D] bf16 (rows = tokens x heads); lse1, lse2, lse_out [rows] fp32 (natural log; -inf = empty partial).
__global__ void __launch_bounds__(128) merge_states_kernel(const __nv_bfloat16* __restrict__ o1, const float* __restrict__ l1,
                                                          const __nv_bfloat16* __restrict__ o2, const float* __restrict__ l2,
                                                          __nv_bfloat16* __restrict__ out, float* __restrict__ lse_out, int D) {
  pdl_wait(); pdl_trigger();
  const long long r = blockIdx.x;
  const float a = l1[r], b = l2[r], m = fmaxf(a, b);
  const float ea = (a == -INFINITY) ? 0.f : __expf(a - m), eb = (b == -INFINITY) ? 0.f : __expf(b - m);
  const float den = ea + eb, wa = den > 0.f ? ea / den : 0.f, wb = den > 0.f ? eb / den : 0.f;
  for (int c = threadIdx.x * 2; c < D; c += blockDim.x * 2) {
    const float2 x = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(o1 + r * D + c));
    const float2 y = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(o2 + r * D + c));
    *reinterpret_cast<uint32_t*>(out + r * D + c) = pack_bf16x2(wa * x.x + wb * y.x, wa * x.y + wb * y.y);
  }
  if (threadIdx.x == 0) lse_out[r] = den > 0.f ? m + __logf(den) : -INFINITY;
}

}  // namespace ne

using namespace ne;

extern "C" int ne_rmsnorm(const void* x, long long x_ld, const void* res_in, const void* w, void* out, long long out_ld, void* res_out,
                          void* q, float* sc, int sc_ld, int T, int H, float eps, float w_off, cudaStream_t st) {
  if (T <= 0) return 0;
  if (H % 8 != 0 || (q && H % 128 != 0) || x_ld % 8 != 0) return 1001;
  size_t smem = (size_t)H * sizeof(float);
  if (smem > 48 * 1024) {
    static bool done = false;
    if (!done) { cudaFuncSetAttribute(rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); done = true; }
  }
  return (int)launch_pdl(rmsnorm_kernel, dim3(T), dim3(256), smem, st, (const __nv_bfloat16*)x, x_ld, (const __nv_bfloat16*)res_in, (const __nv_bfloat16*)w,
                                       (__nv_bfloat16*)out, out_ld, (__nv_bfloat16*)res_out, (uint8_t*)q, sc, sc_ld, H, eps, w_off, g_scale_pow2);
}

extern "C" int ne_quant_1x128(const void* x, long long x_ld, void* q, float* sc, int sc_ld, int T, int K, cudaStream_t st) {
  if (T <= 0) return 0;
  if (K % 128 != 0 || x_ld % 4 != 0) return 1001;
  long long warps = (long long)T * (K / 128);
  int blocks = (int)((warps + 7) / 8);
  return (int)launch_pdl(quant_1x128_kernel, dim3(blocks), dim3(256), 0, st, (const __nv_bfloat16*)x, x_ld, (uint8_t*)q, sc, sc_ld, T, K, g_scale_pow2);
}

extern "C" int ne_act_mul(const void* x, void* y, void* q, float* sc, int sc_ld, long long sc_gs, const int* rows_valid, const int* row_start,
                          int groups, int rows, int I, int act, float p0, float p1, cudaStream_t st);
extern "C" int ne_silu_mul(const void* x, void* y, void* q, float* sc, int sc_ld, long long sc_gs, const int* rows_valid, const int* row_start,
                           int groups, int rows, int I, cudaStream_t st) {
  return ne_act_mul(x, y, q, sc, sc_ld, sc_gs, rows_valid, row_start, groups, rows, I, 0, 0.f, 0.f, st);
}
// the same kernel with the gated activation chosen by `act` (see glu_act)
extern "C" int ne_act_mul(const void* x, void* y, void* q, float* sc, int sc_ld, long long sc_gs, const int* rows_valid, const int* row_start,
                          int groups, int rows, int I, int act, float p0, float p1, cudaStream_t st) {
  if (groups <= 0 || rows <= 0) return 0;
  if (act < 0 || act > 3 || (act != 0 && !(p0 > 0.f))) return 1001;
  if (I % 128 != 0) return 1001;
  long long warps = (long long)groups * rows * (I / 128);
  long long want = (warps + 7) / 8;
  int blocks = (int)(want < 148 * 8 ? want : 148 * 8);
  return (int)launch_pdl(silu_mul_kernel, dim3(blocks), dim3(256), 0, st, (const __nv_bfloat16*)x, (__nv_bfloat16*)y, (uint8_t*)q, sc, sc_ld, sc_gs, rows_valid, row_start, groups, rows, I, act, p0, p1, g_scale_pow2);
}

extern "C" int ne_rope(const void* x, long long row_stride, int head_stride, void* y, long long y_row_stride, int y_head_stride, int heads,
                       int off, int D, const long long* positions, const float* cache, int interleaved, int T, cudaStream_t st) {
  if (T <= 0) return 0;
  long long total = (long long)T * heads * (D / 2);
  return (int)launch_pdl(rope_kernel, dim3((int)((total + 255) / 256)), dim3(256), 0, st, (const __nv_bfloat16*)x, row_stride, head_stride, (__nv_bfloat16*)y, y_row_stride,
                                                          y_head_stride, heads, off, D, positions, cache, interleaved, T);
}

extern "C" int ne_mla_kv_store(const void* ckv, long long ckv_ld, const void* kpe, long long kpe_ld, void* cache, const long long* slots,
                               int T, int R, int rope, int fp8, cudaStream_t st) {
  if (T <= 0) return 0;
  if (R % 2 || rope % 2) return 1001;
  mla_kv_store_kernel<<<(T + 7) / 8, 256, 0, st>>>((const __nv_bfloat16*)ckv, ckv_ld, (const __nv_bfloat16*)kpe, kpe_ld, cache, slots, T, R, rope, fp8);
  return (int)cudaGetLastError();
}

extern "C" int ne_mla_kv_prepare(const void* kv, long long kv_ld, const void* w, float eps, const long long* positions, const float* rope_cache,
                                 void* cache, const long long* slots, int T, int R, int rope, int fp8, cudaStream_t st) {
  if (T <= 0) return 0;
  if (R % 2 || rope % 2 || kv_ld % 2) return 1001;
  return (int)launch_pdl(mla_kv_prepare_kernel, dim3((T + 7) / 8), dim3(256), 0, st, (const __nv_bfloat16*)kv, kv_ld, (const __nv_bfloat16*)w, eps, positions, rope_cache, cache, slots,
                                                     T, R, rope, fp8);
}

extern "C" int ne_mla_q_finalize(const void* q_lat, const void* q_pe, long long pe_row_stride, int pe_head_stride, const long long* positions,
                                 const float* rope_cache, void* q8, int T, int H, int R, int rope, cudaStream_t st) {
  if (T <= 0) return 0;
  if (R % 8 || rope % 2 || pe_row_stride % 2 || pe_head_stride % 2) return 1001;
  long long warps = (long long)T * H;
  return (int)launch_pdl(mla_q_finalize_kernel, dim3((unsigned)((warps + 7) / 8)), dim3(256), 0, st, (const __nv_bfloat16*)q_lat, (const __nv_bfloat16*)q_pe, pe_row_stride, pe_head_stride,
                                                                     positions, rope_cache, (uint8_t*)q8, T, H, R, rope);
}

extern "C" int ne_add(const void* a, const void* b, void* y, long long n, cudaStream_t st) {
  if (n <= 0) return 0;
  if (n % 8) return 1001;
  return (int)launch_pdl(add_kernel, dim3((int)((n / 8 + 255) / 256)), dim3(256), 0, st, (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (__nv_bfloat16*)y, n);
}


extern "C" int ne_gqa_qkv_prepare(const void* qkv, long long ld, int Hq, int Hkv, int D, const void* qw, const void* kw, float eps, float w_offset,
                                  const long long* positions, const float* rope_cache, void* q_out, void* k_cache, void* v_cache,
                                  const long long* slots, int T, cudaStream_t st) {
  if (T <= 0) return 0;
  if ((D != 128 && D != 256) || ld % 2) return 1001;
  const long long warps = (long long)T * (Hq + 2 * Hkv);
  const dim3 grid((unsigned)((warps + 7) / 8));
  if (D == 128)
    return (int)launch_pdl(gqa_qkv_prepare_kernel<128>, grid, dim3(256), 0, st, (const __nv_bfloat16*)qkv, ld, Hq, Hkv, (const __nv_bfloat16*)qw,
                           (const __nv_bfloat16*)kw, eps, w_offset, positions, rope_cache, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache,
                           (__nv_bfloat16*)v_cache, slots, T);
  return (int)launch_pdl(gqa_qkv_prepare_kernel<256>, grid, dim3(256), 0, st, (const __nv_bfloat16*)qkv, ld, Hq, Hkv, (const __nv_bfloat16*)qw,
                         (const __nv_bfloat16*)kw, eps, w_offset, positions, rope_cache, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache,
                         (__nv_bfloat16*)v_cache, slots, T);
}

extern "C" int ne_gqa_kv_store(const void* k, const void* v, long long k_ld, long long v_ld, void* k_cache, void* v_cache, const long long* slots,
                               int T, int row_elems, cudaStream_t st) {
  if (T <= 0) return 0;
  if (row_elems % 8 || k_ld % 8 || v_ld % 8) return 1001;
  return (int)launch_pdl(gqa_kv_store_kernel, dim3(T), dim3(256), 0, st, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, k_ld, v_ld,
                         (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, slots, T, row_elems);
}

extern "C" int ne_gelu(const void* x, void* y, long long n, int tanh_form, cudaStream_t st) {
  if (n <= 0) return 0;
  return (int)launch_pdl(gelu_kernel, dim3((unsigned)((n + 2047) / 2048)), dim3(256), 0, st, (const __nv_bfloat16*)x, (__nv_bfloat16*)y, n, tanh_form);
}

extern "C" int ne_layernorm(const void* x, long long ld, const void* w, const void* b, float eps, void* y, long long rows, int D, cudaStream_t st) {
  if (rows <= 0) return 0;
  return (int)launch_pdl(layernorm_kernel, dim3((unsigned)((rows + 7) / 8)), dim3(256), 0, st, (const __nv_bfloat16*)x, ld, (const __nv_bfloat16*)w,
                         (const __nv_bfloat16*)b, eps, (__nv_bfloat16*)y, rows, D);
}

extern "C" int ne_merge_states(const void* o1, const float* l1, const void* o2, const float* l2, void* out, float* lse_out, long long rows, int D,
                               cudaStream_t st) {
  if (rows <= 0) return 0;
  if (D % 2) return 1001;
  return (int)launch_pdl(merge_states_kernel, dim3((unsigned)rows), dim3(128), 0, st, (const __nv_bfloat16*)o1, l1, (const __nv_bfloat16*)o2, l2,
                         (__nv_bfloat16*)out, lse_out, D);
}
