// Gated delta-net linear attention (Qwen3.5 family): the memory-bound pieces.
//   * causal depthwise convolution + SiLU over ragged sequences with a carried window of the last K-1 inputs per sequence
//   * the recurrent delta rule: one CTA per (sequence, value head) keeps the whole [Dv, Dk] fp32 state in registers, walks the
//     sequence's new tokens, and applies the gated RMSNorm to each output row before it leaves the SM.  A decode step reads
//     and writes the state exactly once (the op's floor: 2 * Dv * Dk * 4 bytes per head), everything else is a few KB.
//   * gated RMSNorm alone, for outputs produced by the chunked (matrix-product) prefill form
// Long prefill sequences run the chunked form on batched matrix products; this kernel serves decode, verification and short chunks.
// Replaces in the reference: layers/backends/delta_net/components/conv.py (causal_conv1d calls and the naive conv),
// components/recurrence.py:100-200, components/output.py:17-62, triton/fla/fused_recurrent.py, triton/generic/rmsnorm_gated.py.
#include "ptx.cuh"

namespace ne {

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }

// grid = (T, ceil(C / (2 * blockDim))); one token per blockIdx.x.  window [S, K-1, C] holds the K-1 inputs before the chunk.
// fused_state != 0 (every sequence contributes exactly one token): the same thread that read a channel's window shifts it.
__global__ void __launch_bounds__(256) gdn_conv_kernel(const __nv_bfloat16* __restrict__ x, long long x_ld, const __nv_bfloat16* __restrict__ w,
                                                      __nv_bfloat16* __restrict__ window, const int* __restrict__ slots,
                                                      const int* __restrict__ cu, const int* __restrict__ fresh, __nv_bfloat16* __restrict__ y,
                                                      long long y_ld, int B, int C, int K, int fused_state) {
  pdl_wait(); pdl_trigger();      // dependent launch: nothing above this line touches global memory
  __shared__ int s_seq;
  const int t = blockIdx.x;
  if (threadIdx.x == 0) {
    int lo = 0, hi = B - 1;                       // last sequence whose start is <= t (empty sequences share a start: take the last)
    while (lo < hi) { int mid = (lo + hi + 1) >> 1; if (cu[mid] <= t) lo = mid; else hi = mid - 1; }
    s_seq = lo;
  }
  __syncthreads();
  const int seq = s_seq;
  const int start = cu[seq], p = t - start;
  const bool is_fresh = fresh[seq] != 0;
  const int slot = slots[seq];
  if (!NE_INDEX_OK(slot, BK_STATE_SLOTS, 21, __LINE__)) return;
  __nv_bfloat16* win = window + (long long)slot * (K - 1) * C;
  for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * 2; c < C; c += gridDim.y * blockDim.x * 2) {
    float acc0 = 0.f, acc1 = 0.f;
    float in0[8], in1[8];                         // K <= 8
    for (int j = 0; j < K; j++) {
      int src = p - (K - 1) + j;                  // position inside the chunk of tap j
      uint32_t u = 0;
      if (src >= 0) u = *reinterpret_cast<const uint32_t*>(x + (long long)(start + src) * x_ld + c);
      else if (!is_fresh) u = *reinterpret_cast<const uint32_t*>(win + (long long)(src + K - 1) * C + c);
      float2 f = unpack_bf16x2(u);
      in0[j] = f.x; in1[j] = f.y;
      acc0 += f.x * __bfloat162float(w[(long long)c * K + j]);
      acc1 += f.y * __bfloat162float(w[(long long)(c + 1) * K + j]);
    }
    *reinterpret_cast<uint32_t*>(y + (long long)t * y_ld + c) = pack_bf16x2(silu_f(acc0), silu_f(acc1));
    if (fused_state)
      for (int j = 1; j < K; j++) *reinterpret_cast<uint32_t*>(win + (long long)(j - 1) * C + c) = pack_bf16x2(in0[j], in1[j]);
  }
}

// grid = (B, ceil(C / (2 * blockDim))): new window of each sequence = the last K-1 inputs (old window entries where the chunk is shorter).
__global__ void __launch_bounds__(256) gdn_conv_state_kernel(const __nv_bfloat16* __restrict__ x, long long x_ld, __nv_bfloat16* __restrict__ window,
                                                            const int* __restrict__ slots, const int* __restrict__ cu,
                                                            const int* __restrict__ fresh, int C, int K) {
  pdl_wait(); pdl_trigger();      // dependent launch: nothing above this line touches global memory
  const int seq = blockIdx.x;
  const int start = cu[seq], n = cu[seq + 1] - start;
  if (n <= 0) return;
  const bool is_fresh = fresh[seq] != 0;
  if (!NE_INDEX_OK(slots[seq], BK_STATE_SLOTS, 21, __LINE__)) return;
  __nv_bfloat16* win = window + (long long)slots[seq] * (K - 1) * C;
  for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * 2; c < C; c += gridDim.y * blockDim.x * 2) {
    uint32_t nw[8];
    for (int j = 0; j < K - 1; j++) {
      int src = n - (K - 1) + j;
      uint32_t u = 0;
      if (src >= 0) u = *reinterpret_cast<const uint32_t*>(x + (long long)(start + src) * x_ld + c);
      else if (!is_fresh) u = *reinterpret_cast<const uint32_t*>(win + (long long)(src + K - 1) * C + c);
      nw[j] = u;
    }
    for (int j = 0; j < K - 1; j++) *reinterpret_cast<uint32_t*>(win + (long long)j * C + c) = nw[j];
  }
}

// grid = (Hv * (Dv / (NW * R)), B), NW warps.  Warp w of a CTA owns R rows of the [Dv, Dk = 32E] state; a lane holds elements
// {e*32 + lane} of each row.  Per token: S *= exp(g); u = beta * (v - S k); S += u k^T; o = S q, evaluated from the two
// dot products S_old.k and S_old.q taken in one pass (o = exp(g) S_old.q + u (k.q)).  Sequences of at least `skip_len` new tokens
// are left to the chunked form.  kFuseNorm (the CTA holds the whole head): the gated RMSNorm is applied here and `out` is
// bf16; otherwise several small CTAs share a head - more CTAs per SM overlap their load / compute / store phases better at
// the 128 x 128 state size - and `out` receives the raw fp32 rows for the separate gated norm kernel.
// kVecGate (Kimi delta attention, reference layers/backends/delta_net/kda.py:300-370): the log-decay is a vector over the key
// dimension, `a` is [T, Hv * Dk] with `dt_bias` of the same width, and the gate is either -exp(A) softplus(a + bias) or, with a
// lower bound L < 0, L * sigmoid(exp(A) (a + bias)).  Row r of the state then decays element by element.
template <int E, int R, int NW, bool kFuseNorm, bool kVecGate>
__global__ void __launch_bounds__(32 * NW) gdn_step_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                                         const __nv_bfloat16* __restrict__ v, long long qk_ld, long long v_ld,
                                                         const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b, long long ab_ld,
                                                         const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                                                         float* __restrict__ state, const int* __restrict__ slots, const int* __restrict__ cu,
                                                         const int* __restrict__ fresh, const __nv_bfloat16* __restrict__ z, long long z_ld,
                                                         const __nv_bfloat16* __restrict__ norm_w, float eps, void* __restrict__ out,
                                                         long long out_ld, int Hv, int Dv, int rep, int skip_len, float lower_bound) {
  pdl_wait(); pdl_trigger();      // dependent launch: nothing above this line touches global memory
  constexpr int Dk = 32 * E, kRowsPerCta = NW * R;
  __shared__ float s_o[kFuseNorm ? kRowsPerCta : 1];
  __shared__ float s_red[NW];
  const int bph = Dv / kRowsPerCta;                    // CTAs per head
  const int h = blockIdx.x / bph, seq = blockIdx.y, hk = h / rep;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = (blockIdx.x % bph) * kRowsPerCta + warp * R;
  const int start = cu[seq], n = cu[seq + 1] - start;
  if (n <= 0 || n >= skip_len) return;
  if (!NE_INDEX_OK(slots[seq], BK_STATE_SLOTS, 21, __LINE__)) return;
  float* S_g = state + (((long long)slots[seq] * Hv + h) * Dv + row0) * Dk;
  float S[R][E];
  if (fresh[seq]) {
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
      for (int e = 0; e < E; e++) S[r][e] = 0.f;
  } else {
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
      for (int e = 0; e < E; e++) S[r][e] = S_g[r * Dk + e * 32 + lane];
  }
  const float neg_A = -__expf(A_log[h]), dtb = kVecGate ? 0.f : dt_bias[h];
  const float qscale = rsqrtf((float)Dk);
  // Inputs of token i + 1 are fetched while token i is computed: a sequence's tokens are strictly serial, so an exposed global
  // load per step (about a microsecond) would otherwise be most of a step of a long prompt chunk.
  float dtv[kVecGate ? E : 1];
  if (kVecGate) {
#pragma unroll
    for (int e = 0; e < E; e++) dtv[e] = dt_bias[h * Dk + e * 32 + lane];
  }
  __nv_bfloat16 rk[E], rq[E], ra[kVecGate ? E : 1], rv[R], rb;
  auto fetch = [&](long long t) {
#pragma unroll
    for (int e = 0; e < E; e++) {
      rk[e] = k[t * qk_ld + hk * Dk + e * 32 + lane];
      rq[e] = q[t * qk_ld + hk * Dk + e * 32 + lane];
      if (kVecGate) ra[e] = a[t * (long long)Hv * Dk + h * Dk + e * 32 + lane];
    }
    if (!kVecGate) ra[0] = a[t * ab_ld + h];
    rb = b[t * ab_ld + h];
#pragma unroll
    for (int r = 0; r < R; r++) rv[r] = v[t * v_ld + h * Dv + row0 + r];
  };
  fetch(start);
  for (int i = 0; i < n; i++) {
    const long long t = start + i;
    float kf[E], qf[E], af[kVecGate ? E : 1], vf[R], kk = 0.f, qq = 0.f, kq = 0.f;
#pragma unroll
    for (int e = 0; e < E; e++) {
      kf[e] = __bfloat162float(rk[e]);
      qf[e] = __bfloat162float(rq[e]);
      if (kVecGate) af[e] = __bfloat162float(ra[e]);
      kk += kf[e] * kf[e]; qq += qf[e] * qf[e];
    }
    if (!kVecGate) af[0] = __bfloat162float(ra[0]);
    const float bf = __bfloat162float(rb);
#pragma unroll
    for (int r = 0; r < R; r++) vf[r] = __bfloat162float(rv[r]);
    if (i + 1 < n) fetch(t + 1);
    kk = warp_sum(kk); qq = warp_sum(qq);
    const float kn = rsqrtf(kk + 1e-6f), qn = rsqrtf(qq + 1e-6f) * qscale;
#pragma unroll
    for (int e = 0; e < E; e++) { kf[e] *= kn; qf[e] *= qn; kq += kf[e] * qf[e]; }
    kq = warp_sum(kq);
    const float beta = 1.f / (1.f + __expf(-bf));
    float o[R];
    if (kVecGate) {
      // `a` rows are Hv * Dk wide here and `b` rows Hv wide; ab_ld is the row stride of `b`, a's is Hv * Dk
      float dec[E], kd[E], qd[E];
#pragma unroll
      for (int e = 0; e < E; e++) {
        const float x = af[e] + dtv[e];
        const float gl = lower_bound < 0.f ? lower_bound / (1.f + __expf(neg_A * x))          // L * sigmoid(exp(A) x)
                                           : neg_A * (x > 20.f ? x : log1pf(__expf(x)));
        dec[e] = __expf(gl); kd[e] = dec[e] * kf[e]; qd[e] = dec[e] * qf[e];
      }
#pragma unroll
      for (int r = 0; r < R; r++) {
        float pk = 0.f, pq = 0.f;
#pragma unroll
        for (int e = 0; e < E; e++) { pk += S[r][e] * kd[e]; pq += S[r][e] * qd[e]; }
        pk = warp_sum(pk); pq = warp_sum(pq);
        const float u = beta * (vf[r] - pk);
#pragma unroll
        for (int e = 0; e < E; e++) S[r][e] = dec[e] * S[r][e] + u * kf[e];
        o[r] = pq + u * kq;
      }
    } else {
      const float av = af[0] + dtb;
      const float sp = av > 20.f ? av : log1pf(__expf(av));
      const float decay = __expf(neg_A * sp);
#pragma unroll
      for (int r = 0; r < R; r++) {
        float pk = 0.f, pq = 0.f;
#pragma unroll
        for (int e = 0; e < E; e++) { pk += S[r][e] * kf[e]; pq += S[r][e] * qf[e]; }
        pk = warp_sum(pk); pq = warp_sum(pq);
        const float u = beta * (vf[r] - decay * pk);
#pragma unroll
        for (int e = 0; e < E; e++) S[r][e] = decay * S[r][e] + u * kf[e];
        o[r] = decay * pq + u * kq;
      }
    }
    if (!kFuseNorm) {
      float* orow = reinterpret_cast<float*>(out) + t * out_ld + h * Dv + row0;
      if (lane == 0) {
#pragma unroll
        for (int r = 0; r < R; r++) orow[r] = o[r];
      }
      continue;
    }
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < R; r++) s_o[warp * R + r] = o[r];
    }
    __syncthreads();
    // gated RMSNorm over the head's Dv outputs (the CTA holds them all: kRowsPerCta == Dv <= blockDim.x)
    float val = (int)threadIdx.x < Dv ? s_o[threadIdx.x] : 0.f;
    float ss = warp_sum(val * val);
    if (lane == 0) s_red[warp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int wv = 0; wv < NW; wv++) tot += s_red[wv];
    if ((int)threadIdx.x < Dv) {
      const int d = threadIdx.x;
      float xn = __bfloat162float(__float2bfloat16(val * rsqrtf(tot / (float)Dv + eps)));
      float y = __bfloat162float(__float2bfloat16(__bfloat162float(norm_w[d]) * xn));
      float zg = __bfloat162float(__float2bfloat16(silu_f(__bfloat162float(z[t * z_ld + h * Dv + d]))));
      reinterpret_cast<__nv_bfloat16*>(out)[t * out_ld + h * Dv + d] = __float2bfloat16(y * zg);
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < R; r++)
#pragma unroll
    for (int e = 0; e < E; e++) S_g[r * Dk + e * 32 + lane] = S[r][e];
}

// one warp per row: out = w * bf16(rmsnorm(x)) * bf16(silu(z)); rows listed by [row_begin, row_end) ranges are handled by the caller.
__global__ void __launch_bounds__(256) rmsnorm_gated_kernel(const float* __restrict__ x, const __nv_bfloat16* __restrict__ z, long long z_ld,
                                                           const __nv_bfloat16* __restrict__ w, float eps, __nv_bfloat16* __restrict__ out,
                                                           long long out_ld, long long rows, int heads, int D, int sigmoid_fp32) {
  pdl_wait(); pdl_trigger();      // dependent launch: nothing above this line touches global memory
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const long long t = row / heads;
  const int h = (int)(row % heads);
  const float* xr = x + row * D;
  float ss = 0.f;
  for (int d = lane; d < D; d += 32) { float f = xr[d]; ss += f * f; }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / (float)D + eps);
  if (sigmoid_fp32) {        // x * rstd * w * sigmoid(z) in fp32, one rounding (reference kernel/triton/generic/k3_output_norm.py:40)
    for (int d = lane; d < D; d += 32)
      out[t * out_ld + h * D + d] = __float2bfloat16(xr[d] * rstd * __bfloat162float(w[d]) / (1.f + __expf(-__bfloat162float(z[t * z_ld + h * D + d]))));
    return;
  }
  for (int d = lane; d < D; d += 32) {
    float xn = __bfloat162float(__float2bfloat16(xr[d] * rstd));
    float y = __bfloat162float(__float2bfloat16(__bfloat162float(w[d]) * xn));
    float zg = __bfloat162float(__float2bfloat16(silu_f(__bfloat162float(z[t * z_ld + h * D + d]))));
    out[t * out_ld + h * D + d] = __float2bfloat16(y * zg);
  }
}

// out = o * sigmoid(gate); o, out [T, heads, D] contiguous, gate a strided view (row and head strides in elements); two columns per thread
__global__ void __launch_bounds__(256) sigmoid_gate_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ gate, long long g_row,
                                                          long long g_head, __nv_bfloat16* __restrict__ out, long long pairs, int heads, int D) {
  pdl_wait(); pdl_trigger();      // dependent launch: nothing above this line touches global memory
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= pairs) return;
  const int half = D / 2;
  const int d = (int)(i % half) * 2;
  const long long th = i / half;
  const int h = (int)(th % heads);
  const long long t = th / heads;
  float2 ov = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(o + th * D + d));
  const __nv_bfloat16* gp = gate + t * g_row + h * g_head + d;
  float g0 = __bfloat162float(gp[0]), g1 = __bfloat162float(gp[1]);
  *reinterpret_cast<uint32_t*>(out + th * D + d) = pack_bf16x2(ov.x / (1.f + __expf(-g0)), ov.y / (1.f + __expf(-g1)));
}

}  // namespace ne

using namespace ne;

extern "C" int ne_sigmoid_gate(const void* o, const void* gate, long long g_row, long long g_head, void* out, long long T, int heads, int D, cudaStream_t st) {
  long long pairs = T * heads * (D / 2);
  if (pairs <= 0) return 0;
  if (D % 2) return 1001;
  return (int)launch_pdl(sigmoid_gate_kernel, dim3((unsigned)((pairs + 255) / 256)), dim3(256), 0, st, (const __nv_bfloat16*)o, (const __nv_bfloat16*)gate, g_row, g_head,
                                                                      (__nv_bfloat16*)out, pairs, heads, D);
}

extern "C" int ne_gdn_conv(const void* x, long long x_ld, const void* w, void* window, const int* slots, const int* cu, const int* fresh, void* y,
                           long long y_ld, int T, int B, int C, int K, int uniform_one, cudaStream_t st) {
  if (T <= 0 || B <= 0) return 0;
  if (C % 2 || x_ld % 2 || y_ld % 2 || K < 2 || K > 8) return 1001;
  int gy = (C / 2 + 255) / 256;
  if (gy > 8) gy = 8;
  cudaError_t e = launch_pdl(gdn_conv_kernel, dim3(T, gy), dim3(256), 0, st, (const __nv_bfloat16*)x, x_ld, (const __nv_bfloat16*)w,
                             (__nv_bfloat16*)window, slots, cu, fresh, (__nv_bfloat16*)y, y_ld, B, C, K, uniform_one);
  if (e != cudaSuccess || uniform_one) return (int)e;
  // the window update starts only after the convolution above has read the old window: its writes follow its own dependency wait
  return (int)launch_pdl(gdn_conv_state_kernel, dim3(B, gy), dim3(256), 0, st, (const __nv_bfloat16*)x, x_ld, (__nv_bfloat16*)window, slots, cu,
                         fresh, C, K);
}

// raw_out != 0: `out` is fp32 [T, Hv, Dv] without the gated norm (the caller runs ne_rmsnorm_gated); the 128 x 128 state size
// always takes that form.  Returns 0, an argument error, or 1 when the caller asked for the fused form at a size that has none.
extern "C" int ne_gdn_step_raw_only(int Dk, int Dv) { return (Dk == 128 && Dv == 128) ? 1 : 0; }
extern "C" int ne_gdn_step(const void* q, const void* k, const void* v, long long qk_ld, long long v_ld, const void* a, const void* b, long long ab_ld,
                           const float* A_log, const float* dt_bias, float* state, const int* slots, const int* cu, const int* fresh,
                           const void* z, long long z_ld, const void* norm_w, float eps, void* out, long long out_ld, int B, int Hk, int Hv,
                           int Dk, int Dv, int skip_len, int raw_out, int vec_gate, float lower_bound, cudaStream_t st) {
  if (B <= 0) return 0;
  if (Hv % Hk) return 1001;
  const int rep = Hv / Hk;
  if (vec_gate && !(Dk == 128 && Dv == 128 && raw_out)) return 1001;
#define NE_GDN_LAUNCH(E_, R_, NW_, FUSE_, VEC_)                                                                                                 \
  launch_pdl(gdn_step_kernel<E_, R_, NW_, FUSE_, VEC_>, dim3(Hv * (Dv / (NW_ * R_)), B), dim3(32 * NW_), 0, st,                                \
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, qk_ld, v_ld, (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, \
      ab_ld, A_log, dt_bias, state, slots, cu, fresh, (const __nv_bfloat16*)z, z_ld, (const __nv_bfloat16*)norm_w, eps, out, out_ld, Hv, Dv, rep, \
      skip_len, lower_bound)
  if (Dk == 128 && Dv == 128) { if (!raw_out) return 1001; if (vec_gate) NE_GDN_LAUNCH(4, 8, 4, false, true); else NE_GDN_LAUNCH(4, 8, 4, false, false); }
  else if (raw_out) return 1001;
  else if (Dk == 128 && Dv == 64) NE_GDN_LAUNCH(4, 8, 8, true, false);
  else if (Dk == 64 && Dv == 64) NE_GDN_LAUNCH(2, 8, 8, true, false);
  else if (Dk == 32 && Dv == 32) NE_GDN_LAUNCH(1, 4, 8, true, false);
  else return 1001;
#undef NE_GDN_LAUNCH
  return (int)cudaGetLastError();
}

extern "C" int ne_rmsnorm_gated(const float* x, const void* z, long long z_ld, const void* w, float eps, void* out, long long out_ld, long long tokens,
                                int heads, int D, int sigmoid_fp32, cudaStream_t st) {
  long long rows = tokens * heads;
  if (rows <= 0) return 0;
  return (int)launch_pdl(rmsnorm_gated_kernel, dim3((unsigned)((rows + 7) / 8)), dim3(256), 0, st, x, (const __nv_bfloat16*)z, z_ld, (const __nv_bfloat16*)w, eps, (__nv_bfloat16*)out,
                                                                  out_ld, rows, heads, D, sigmoid_fp32);
}
