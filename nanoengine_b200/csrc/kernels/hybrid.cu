// Residual-stream kernels of the hybrid delta-attention families.
//
//  * attn_res_kernel: block attention residuals (Kimi-K3).  The layer input is a softmax mixture over the frozen block sums in
//    the bank and the running sum since the last block boundary, scored by an RMS-normalised dot product with one weight
//    vector, followed by the layer's RMSNorm.  One CTA per token: pass 1 takes the sum of squares and the score dot product of
//    every candidate row, pass 2 re-reads the rows (L1 / L2 hits), mixes them in registers and normalises.
//    Replaces in the reference: kernel/jit/sgl/csrc/kimi_k3/attn_res/fused_tma.cuh:444 and
//    kernel/triton/kimi_k3/attn_residual.py:17-140 (two launches: scores, combine).
//  * mhc_pre_kernel / mhc_post_kernel: manifold-constrained hyper-connections (GLM5-next).  The hidden state is `h` parallel
//    streams; before a sub-layer the streams are contracted with sigmoid weights, after it the sub-layer output is spread
//    back with a second set of weights and the streams are mixed by a Sinkhorn-normalised h x h matrix.  All 2h + h*h
//    coefficients of a token come from one product of the flattened streams with a [(2+h)h, h*D] matrix, which runs as a
//    tensor-core GEMM in front of mhc_mix_kernel.
//    Replaces in the reference: models/glm5_next/glm5_next.py:27-99 (PyTorch modules).
#include "ptx.cuh"

namespace ne {

constexpr int kResMaxRows = 17;       // bank rows + the running prefix
constexpr int kResMaxChunks = 4;      // 8-element chunks per thread: D <= 256 * 8 * 4 = 8192

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* f) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float* f) {
  *reinterpret_cast<uint4*>(p) = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
}

// prefix [T, D] (row stride p_ld), bank [T, rows, D] (token stride b_ts, row stride b_rs), candidates = bank rows [0, valid) + prefix.
// out = w_out * rmsnorm(bf16(sum_c softmax(score)_c cand_c)); score_c = (cand_c . w_score) * rsqrt(mean(cand_c^2) + eps).
// write_row >= 0: the prefix is also stored into bank row `write_row`.
__global__ void __launch_bounds__(256) attn_res_kernel(const __nv_bfloat16* __restrict__ prefix, long long p_ld, __nv_bfloat16* __restrict__ bank,
                                                      long long b_ts, long long b_rs, int valid, const float* __restrict__ w_score,
                                                      const __nv_bfloat16* __restrict__ w_out, float eps, __nv_bfloat16* __restrict__ out,
                                                      long long o_ld, int D, int write_row) {
  pdl_wait(); pdl_trigger();      // dependent launch: nothing above this line touches global memory
  __shared__ float s_part[8][2 * kResMaxRows];
  __shared__ float s_p[kResMaxRows];
  __shared__ float s_red[8];
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nc = valid + 1, chunks = D / 8;
  const __nv_bfloat16* pr = prefix + (long long)t * p_ld;
  __nv_bfloat16* bk = bank + (long long)t * b_ts;
  for (int c = 0; c < nc; c++) {
    const __nv_bfloat16* row = c < valid ? bk + (long long)c * b_rs : pr;
    float ss = 0.f, dot = 0.f;
    for (int ch = threadIdx.x; ch < chunks; ch += 256) {
      float f[8];
      load8(row + ch * 8, f);
      const float4 w0 = *reinterpret_cast<const float4*>(w_score + ch * 8), w1 = *reinterpret_cast<const float4*>(w_score + ch * 8 + 4);
      const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int j = 0; j < 8; j++) { ss += f[j] * f[j]; dot += f[j] * w[j]; }
    }
    ss = warp_sum(ss); dot = warp_sum(dot);
    if (lane == 0) { s_part[warp][2 * c] = ss; s_part[warp][2 * c + 1] = dot; }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float sc[kResMaxRows], mx = -INFINITY;
    for (int c = 0; c < nc; c++) {
      float ss = 0.f, dot = 0.f;
      for (int w = 0; w < 8; w++) { ss += s_part[w][2 * c]; dot += s_part[w][2 * c + 1]; }
      sc[c] = dot * rsqrtf(ss / (float)D + eps);
      mx = fmaxf(mx, sc[c]);
    }
    float sum = 0.f;
    for (int c = 0; c < nc; c++) { sc[c] = __expf(sc[c] - mx); sum += sc[c]; }
    for (int c = 0; c < nc; c++) s_p[c] = sc[c] / sum;
  }
  __syncthreads();
  float m[kResMaxChunks][8];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < kResMaxChunks; k++) {
    const int ch = threadIdx.x + k * 256;
#pragma unroll
    for (int j = 0; j < 8; j++) m[k][j] = 0.f;
    if (ch < chunks) {
      for (int c = 0; c < nc; c++) {
        const __nv_bfloat16* row = c < valid ? bk + (long long)c * b_rs : pr;
        float f[8];
        load8(row + ch * 8, f);
        const float p = s_p[c];
#pragma unroll
        for (int j = 0; j < 8; j++) m[k][j] += p * f[j];
        if (c == valid && write_row >= 0) store8(bk + (long long)write_row * b_rs + ch * 8, f);
      }
#pragma unroll
      for (int j = 0; j < 8; j++) { m[k][j] = __bfloat162float(__float2bfloat16(m[k][j])); ss += m[k][j] * m[k][j]; }
    }
  }
  ss = warp_sum(ss);
  if (lane == 0) s_red[warp] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < 8; w++) tot += s_red[w];
  const float rstd = rsqrtf(tot / (float)D + eps);
#pragma unroll
  for (int k = 0; k < kResMaxChunks; k++) {
    const int ch = threadIdx.x + k * 256;
    if (ch < chunks) {
      float w[8], o[8];
      load8(w_out + ch * 8, w);
#pragma unroll
      for (int j = 0; j < 8; j++) o[j] = m[k][j] * rstd * w[j];
      store8(out + (long long)t * o_ld + ch * 8, o);
    }
  }
}

// ---- hyper-connections -------------------------------------------------------------------------------------------------
constexpr int kHcMaxM = 24;     // (2 + h) * h for h <= 4

// The coefficient product mixes[t, m] = x[t, :] . fn[m, :] over the h*D flattened streams runs on the tensor cores as one
// bf16 GEMM: fn (fp32 in the checkpoint) is split into a bf16 head and a bf16 remainder, stacked as 2M weight rows, so the two
// partial products add up to the fp32 product to ~2^-17 relative (x is bf16 already, accumulation is fp32).  This kernel takes
// the GEMM's [T, ldm] fp32 output (columns [0, M) head, [M, 2M) remainder) and does everything else, one CTA per token: sum of
// squares of the streams, sigmoid / softmax / Sinkhorn coefficients in one thread, stream contraction y = sum_i pre_i x_i
// (the second pass over the token's h*D values hits L1 / L2).
// x [T, h, D] bf16 contiguous; base [(2+h)h]; scale [3].  y [T, D], post [T, h], comb [T, h, h] bf16 (as the reference rounds them).
__global__ void __launch_bounds__(256) mhc_mix_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ mixes, int ldm,
                                                     const float* __restrict__ base, const float* __restrict__ scale, __nv_bfloat16* __restrict__ y,
                                                     __nv_bfloat16* __restrict__ post, __nv_bfloat16* __restrict__ comb, int h, int D, int iters,
                                                     float eps) {
  pdl_wait(); pdl_trigger();      // dependent launch: nothing above this line touches global memory
  __shared__ float s_red[8];
  __shared__ float s_pre[4];
  const int M = (2 + h) * h, W = h * D;
  const long long t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const __nv_bfloat16* xt = x + t * W;
  float ss = 0.f;
  for (int e = threadIdx.x * 8; e < W; e += 256 * 8) {
    float f[8];
    load8(xt + e, f);
#pragma unroll
    for (int j = 0; j < 8; j++) ss += f[j] * f[j];
  }
  ss = warp_sum(ss);
  if (lane == 0) s_red[warp] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int w = 0; w < 8; w++) tot += s_red[w];
    const float r = rsqrtf(tot / (float)W + eps);
    const float* mr = mixes + t * ldm;
    float mix[kHcMaxM];
    for (int m = 0; m < M; m++) mix[m] = (mr[m] + mr[M + m]) * r;
    for (int i = 0; i < h; i++) {
      const float pre = 1.f / (1.f + __expf(-(mix[i] * scale[0] + base[i]))) + eps;
      s_pre[i] = __bfloat162float(__float2bfloat16(pre));
      post[t * h + i] = __float2bfloat16(2.f / (1.f + __expf(-(mix[h + i] * scale[1] + base[h + i]))));
    }
    float c[4][4];
    for (int i = 0; i < h; i++) {
      float mx = -INFINITY, sum = 0.f;
      for (int j = 0; j < h; j++) { c[i][j] = mix[2 * h + i * h + j] * scale[2] + base[2 * h + i * h + j]; mx = fmaxf(mx, c[i][j]); }
      for (int j = 0; j < h; j++) { c[i][j] = __expf(c[i][j] - mx); sum += c[i][j]; }
      for (int j = 0; j < h; j++) c[i][j] = c[i][j] / sum + eps;
    }
    auto cols = [&]() {
      for (int j = 0; j < h; j++) {
        float sm = 0.f;
        for (int i = 0; i < h; i++) sm += c[i][j];
        for (int i = 0; i < h; i++) c[i][j] /= sm + eps;
      }
    };
    cols();
    for (int it = 1; it < iters; it++) {
      for (int i = 0; i < h; i++) {
        float sm = 0.f;
        for (int j = 0; j < h; j++) sm += c[i][j];
        for (int j = 0; j < h; j++) c[i][j] /= sm + eps;
      }
      cols();
    }
    for (int i = 0; i < h; i++)
      for (int j = 0; j < h; j++) comb[(t * h + i) * h + j] = __float2bfloat16(c[i][j]);
  }
  __syncthreads();
  for (int d = threadIdx.x * 8; d < D; d += 256 * 8) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int i = 0; i < h; i++) {
      float f[8];
      load8(xt + (long long)i * D + d, f);
      const float p = s_pre[i];
#pragma unroll
      for (int j = 0; j < 8; j++) acc[j] += p * f[j];
    }
    store8(y + t * D + d, acc);
  }
}

// out[t, i, :] = post[t, i] * x[t, :] + sum_j comb[t, j, i] * res[t, j, :]
__global__ void __launch_bounds__(256) mhc_post_kernel(const __nv_bfloat16* __restrict__ x, long long x_ld, const __nv_bfloat16* __restrict__ res,
                                                      const __nv_bfloat16* __restrict__ post, const __nv_bfloat16* __restrict__ comb,
                                                      __nv_bfloat16* __restrict__ out, long long T, int h, int D) {
  pdl_wait(); pdl_trigger();      // dependent launch: nothing above this line touches global memory
  const int chunks = D / 8;
  const long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (item >= T * chunks) return;
  const long long t = item / chunks;
  const int ch = (int)(item % chunks);
  float xv[8], r[4][8];
  load8(x + t * x_ld + ch * 8, xv);
  for (int j = 0; j < h; j++) load8(res + (t * h + j) * D + ch * 8, r[j]);
  for (int i = 0; i < h; i++) {
    const float p = __bfloat162float(post[t * h + i]);
    float o[8];
#pragma unroll
    for (int e = 0; e < 8; e++) o[e] = p * xv[e];
    for (int j = 0; j < h; j++) {
      const float c = __bfloat162float(comb[(t * h + j) * h + i]);
#pragma unroll
      for (int e = 0; e < 8; e++) o[e] += c * r[j][e];
    }
    store8(out + (t * h + i) * D + ch * 8, o);
  }
}

// o * sigmoid(g) elementwise over contiguous bf16 rows (output gate of the NoPE MLA layers)
__global__ void __launch_bounds__(256) sigmoid_mul_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ g, long long g_ld,
                                                         __nv_bfloat16* __restrict__ out, long long T, int W) {
  pdl_wait(); pdl_trigger();      // dependent launch: nothing above this line touches global memory
  const int chunks = W / 8;
  const long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (item >= T * chunks) return;
  const long long t = item / chunks;
  const int ch = (int)(item % chunks);
  float a[8], b[8];
  load8(o + t * W + ch * 8, a);
  load8(g + t * g_ld + ch * 8, b);
#pragma unroll
  for (int e = 0; e < 8; e++) a[e] = a[e] / (1.f + __expf(-b[e]));
  store8(out + t * W + ch * 8, a);
}

}  // namespace ne

using namespace ne;

extern "C" int ne_attn_res(const void* prefix, long long p_ld, void* bank, long long b_ts, long long b_rs, int valid, const float* w_score,
                           const void* w_out, float eps, void* out, long long o_ld, int T, int D, int write_row, cudaStream_t st) {
  if (T <= 0) return 0;
  if (D % 8 || D > 256 * 8 * kResMaxChunks || valid < 0 || valid + 1 > kResMaxRows || p_ld % 8 || b_ts % 8 || b_rs % 8 || o_ld % 8) return 1001;
  return (int)launch_pdl(attn_res_kernel, dim3(T), dim3(256), 0, st, (const __nv_bfloat16*)prefix, p_ld, (__nv_bfloat16*)bank, b_ts, b_rs, valid, w_score,
                         (const __nv_bfloat16*)w_out, eps, (__nv_bfloat16*)out, o_ld, D, write_row);
}

extern "C" int ne_mhc_mix(const void* x, const float* mixes, int ldm, const float* base, const float* scale, void* y, void* post, void* comb, int T,
                          int h, int D, int iters, float eps, cudaStream_t st) {
  if (T <= 0) return 0;
  if (h < 1 || h > 4 || D % 8 || ldm < 2 * (2 + h) * h) return 1001;
  return (int)launch_pdl(mhc_mix_kernel, dim3(T), dim3(256), 0, st, (const __nv_bfloat16*)x, mixes, ldm, base, scale, (__nv_bfloat16*)y,
                         (__nv_bfloat16*)post, (__nv_bfloat16*)comb, h, D, iters, eps);
}

extern "C" int ne_mhc_post(const void* x, long long x_ld, const void* res, const void* post, const void* comb, void* out, long long T, int h, int D,
                           cudaStream_t st) {
  if (T <= 0) return 0;
  if (h < 1 || h > 4 || D % 8 || x_ld % 8) return 1001;
  const long long items = T * (D / 8);
  return (int)launch_pdl(mhc_post_kernel, dim3((unsigned)((items + 255) / 256)), dim3(256), 0, st, (const __nv_bfloat16*)x, x_ld, (const __nv_bfloat16*)res,
                         (const __nv_bfloat16*)post, (const __nv_bfloat16*)comb, (__nv_bfloat16*)out, T, h, D);
}

extern "C" int ne_sigmoid_mul(const void* o, const void* g, long long g_ld, void* out, long long T, int W, cudaStream_t st) {
  if (T <= 0) return 0;
  if (W % 8 || g_ld % 8) return 1001;
  const long long items = T * (W / 8);
  return (int)launch_pdl(sigmoid_mul_kernel, dim3((unsigned)((items + 255) / 256)), dim3(256), 0, st, (const __nv_bfloat16*)o, (const __nv_bfloat16*)g, g_ld,
                         (__nv_bfloat16*)out, T, W);
}
