// MoE routing and the token <-> expert-major layout transforms around the grouped GEMMs.
//
//   route    : sigmoid / sqrt-softplus (+ correction bias, group-limited) or softmax top-k with renormalisation and scaling
//   count    : per-expert token counts and each (token, k) pair's slot inside its expert
//   scan     : 128-aligned exclusive prefix over the counts -> row_start[e] (every expert's rows start a GEMM tile)
//   scatter  : write each routed token row into the expert-major buffer, quantising to e4m3 1x128 on the way
//   combine  : out[t] = sum_k w[t,k] * Y[pos[t,k]] (+ shared-expert output), fixed k order -> deterministic
// Everything data-dependent stays on the device, so the whole sequence is CUDA-graph capturable.
//
// Replaces in the reference: jit/sgl/csrc/moe/moe_fused_gate.cuh, triton/generic/fused_topk.py:26-129,
// triton/hopper/fused_moe_v3.py:214-453 (ep_scatter / ep_gather), triton/generic/local_dispatch.py:25-84.
#include "ptx.cuh"

namespace ne {

constexpr int kMaxExperts = 1024;

// one warp per token
__global__ void __launch_bounds__(128) moe_route_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int* __restrict__ idx_out,
                                                       float* __restrict__ w_out, int T, int E, int top_k, int n_group, int topk_group,
                                                       int norm, float scale, int softmax, int planes, int balance_ranks,
                                                       const int* __restrict__ log2phy, const int* __restrict__ logcnt, int max_rep) {
  pdl_wait(); pdl_trigger();      // dependent launch: nothing above this line touches global memory
  __shared__ float s_choice[4][kMaxExperts];
  __shared__ float s_score[4][kMaxExperts];
  __shared__ float s_group[4][64];
  const int wl = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + wl;
  if (t >= T) return;
  float* choice = s_choice[wl]; float* score = s_score[wl]; float* gsc = s_group[wl];
  // the logits may arrive as `planes` partial sums [planes, T, E] (split-K router product)
  for (int e = lane; e < E; e += 32) {
    float v = 0.f;
    for (int p = 0; p < planes; p++) v += logits[((long long)p * T + t) * E + e];
    choice[e] = v;
  }
  const float* lr = choice;
  if (softmax == 1) {
    float m = -INFINITY;
    for (int e = lane; e < E; e += 32) m = fmaxf(m, lr[e]);
    m = warp_max(m);
    float s = 0.f;
    for (int e = lane; e < E; e += 32) { float v = __expf(lr[e] - m); score[e] = v; s += v; }
    s = warp_sum(s);
    float inv = 1.f / s;
    for (int e = lane; e < E; e += 32) { score[e] *= inv; choice[e] = score[e] + (bias ? bias[e] : 0.f); }
  } else {
    // softmax == 2: sqrt(softplus(x)) (DeepSeek-V4), else sigmoid
    for (int e = lane; e < E; e += 32) {
      const float x = lr[e];
      float v = softmax == 2 ? sqrtf(x > 20.f ? x : log1pf(__expf(x))) : 1.f / (1.f + __expf(-x));
      score[e] = v; choice[e] = v + (bias ? bias[e] : 0.f);
    }
  }
  __syncwarp();
  if (n_group > 1) {
    const int gs = E / n_group;
    for (int g = lane; g < n_group; g += 32) {
      float a = -INFINITY, b = -INFINITY;      // two largest of the group
      for (int j = 0; j < gs; j++) { float v = choice[g * gs + j]; if (v > a) { b = a; a = v; } else if (v > b) b = v; }
      gsc[g] = a + b;
    }
    __syncwarp();
    // keep the topk_group best groups (lowest index wins ties); lane g decides for group g
    for (int g = lane; g < n_group; g += 32) {
      int better = 0;
      for (int h = 0; h < n_group; h++) better += (gsc[h] > gsc[g]) || (gsc[h] == gsc[g] && h < g);
      if (better >= topk_group) for (int j = 0; j < gs; j++) choice[g * gs + j] = -INFINITY;
    }
    __syncwarp();
  }
  float wsum = 0.f;
  for (int k = 0; k < top_k; k++) {
    float best = -INFINITY; int bi = E;
    for (int e = lane; e < E; e += 32) { float v = choice[e]; if (v > best) { best = v; bi = e; } }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ob = __shfl_xor_sync(0xffffffffu, best, o); int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (bi >= E) bi = 0;   // every remaining choice is -inf (cannot happen with valid arguments)
    float sv = score[bi];
    wsum += sv;
    if (lane == 0) {
      int phys = bi;
      if (balance_ranks > 0) {
        // load-balance stand-in for random-init routers: expert ids dealt round-robin over the EP ranks, weights kept
        const int i = t * top_k + k, step = E / balance_ranks;
        phys = ((i / balance_ranks) % step + (i % balance_ranks) * step) % E;
      } else if (log2phy) {
        // EPLB: logical expert -> one of its physical replicas, chosen by token so that replicas share the load
        const int cnt = logcnt[bi];
        phys = log2phy[bi * max_rep + (cnt > 1 ? (int)(((unsigned)t * 2654435761u + (unsigned)k * 40503u) >> 8) % cnt : 0)];
      }
      idx_out[(long long)t * top_k + k] = phys; w_out[(long long)t * top_k + k] = sv; choice[bi] = -INFINITY;
    }
    __syncwarp();
  }
  if (lane == 0) {
    float f = (norm ? 1.f / (wsum + 1e-20f) : 1.f) * scale;
    for (int k = 0; k < top_k; k++) w_out[(long long)t * top_k + k] *= f;
  }
}

// slot[t,k] = running index of the pair inside its (local) expert, counts[e] = pairs per expert
__global__ void moe_count_kernel(const int* __restrict__ idx, int* __restrict__ counts, int* __restrict__ slot, int n_pairs, int expert_offset, int E_local) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_pairs) return;
  int e = idx[i] - expert_offset;
  slot[i] = (e >= 0 && e < E_local) ? atomicAdd(&counts[e], 1) : -1;
}

// single CTA: row_start[e] = sum_{e' < e} align(counts[e'], align); row_start[E] = total
__global__ void moe_scan_kernel(const int* __restrict__ counts, int* __restrict__ row_start, int E, int align) {
  __shared__ int s[kMaxExperts + 1];
  for (int e = threadIdx.x; e < E; e += blockDim.x) s[e] = (counts[e] + align - 1) / align * align;
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; e++) { int c = s[e]; s[e] = acc; acc += c; }
    s[E] = acc;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) row_start[e] = s[e];
}

// The two kernels above in one CTA (no zeroed input needed): counts are taken with shared-memory atomics, the aligned
// prefix sums follow, and both tables are written out.  One CTA walks all T * top_k pairs; at 16K tokens that is a few tens
// of microseconds, a small cost against saving two launches and a memset per MoE layer in every decode step.
__global__ void __launch_bounds__(1024) moe_count_scan_kernel(const int* __restrict__ idx, int* __restrict__ counts, int* __restrict__ slot,
                                                             int* __restrict__ row_start, int n_pairs, int expert_offset, int E, int align) {
  pdl_wait(); pdl_trigger();      // dependent launch: nothing above this line touches global memory
  __shared__ int s_cnt[kMaxExperts + 1];
  for (int e = threadIdx.x; e <= E; e += blockDim.x) s_cnt[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int e = idx[i] - expert_offset;
    slot[i] = (e >= 0 && e < E) ? atomicAdd(&s_cnt[e], 1) : -1;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = s_cnt[e];
  __syncthreads();
  if (threadIdx.x < 32) {
    // warp scan over the aligned counts, 32 experts per round
    int carry = 0;
    for (int e0 = 0; e0 < E; e0 += 32) {
      const int e = e0 + (int)threadIdx.x;
      const int c = e < E ? (s_cnt[e] + align - 1) / align * align : 0;
      int incl = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) { const int v = __shfl_up_sync(0xffffffffu, incl, o); if ((int)threadIdx.x >= o) incl += v; }
      if (e < E) row_start[e] = carry + incl - c;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (threadIdx.x == 0) row_start[E] = carry;
  }
}

// One CTA per token: the row is quantised to e4m3 1x128 once (kept in shared memory) and then copied to each of the
// token's local experts; writes pos[t,k] (row in the expert-major buffer, -1 if not local / overflow).
__global__ void __launch_bounds__(256) moe_scatter_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ idx, const int* __restrict__ slot,
                                   const int* __restrict__ row_start, int* __restrict__ pos, __nv_bfloat16* __restrict__ a_bf16,
                                   uint8_t* __restrict__ a_q, float* __restrict__ a_s, int s_ld, int top_k, int H,
                                   int expert_offset, int E_local, int max_rows, int pow2) {
  pdl_wait(); pdl_trigger();      // dependent launch: nothing above this line touches global memory
  extern __shared__ uint8_t s_raw[];
  uint32_t* s_q = reinterpret_cast<uint32_t*>(s_raw);                 // H bytes of e4m3
  float* s_sc = reinterpret_cast<float*>(s_raw + H);                  // H/128 scales
  __shared__ int s_row[64];
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if ((int)threadIdx.x < top_k) {
    const int i = t * top_k + threadIdx.x;
    const int e = idx[i] - expert_offset, sl = slot[i];
    int row = -1;
    if (e >= 0 && e < E_local && sl >= 0) { row = row_start[e] + sl; if (row >= max_rows) row = -1; }
    pos[i] = row; s_row[threadIdx.x] = row;
  }
  const __nv_bfloat16* xr = x + (long long)t * H;
  if (a_q) {
    for (int g = warp; g < H / 128; g += nw) {
      uint2 v = *reinterpret_cast<const uint2*>(xr + g * 128 + lane * 4);
      float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y);
      float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
      amax = fmaxf(warp_max(amax), 1e-10f);
      float is; const float sg = fp8_group_scale(amax, pow2, &is);
      s_q[g * 32 + lane] = pack_e4m3x4(a.x * is, a.y * is, b.x * is, b.y * is);
      if (lane == 0) s_sc[g] = sg;
    }
  }
  __syncthreads();
  for (int k = 0; k < top_k; k++) {
    const int row = s_row[k];
    if (row < 0) continue;
    if (a_q) {
      uint4* dst = reinterpret_cast<uint4*>(a_q + (long long)row * H);
      const uint4* src = reinterpret_cast<const uint4*>(s_q);
      for (int c = threadIdx.x; c < H / 16; c += blockDim.x) dst[c] = src[c];
      for (int g = threadIdx.x; g < H / 128; g += blockDim.x) a_s[(long long)g * s_ld + row] = s_sc[g];
    } else {
      for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) *reinterpret_cast<uint4*>(a_bf16 + (long long)row * H + c) = *reinterpret_cast<const uint4*>(xr + c);
    }
  }
}

// Router logits on CUDA cores with the fp32 gate weight: logits[t, e] = x[t, :] . w[e, :], split along the hidden
// dimension into planes of kRouterCols columns that the routing kernel adds up.  One CTA = 8 tokens x 32 experts x one
// column slice: the tokens' slice sits in shared memory, each warp takes 4 experts, streams each expert's slice with
// eight 16-byte loads in flight per lane and keeps 8 running sums.
constexpr int kRouterCols = 1024;
__global__ void __launch_bounds__(256) router_gemv_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w, float* __restrict__ planes,
                                                         int T, int E, int H) {
  pdl_wait(); pdl_trigger();      // dependent launch: nothing above this line touches global memory
  __shared__ __align__(16) __nv_bfloat16 s_x[8][kRouterCols];
  const int t0 = blockIdx.x * 8, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h0 = blockIdx.z * kRouterCols;
  const int hc = min(kRouterCols, H - h0);                                // multiple of 128
  for (int i = threadIdx.x * 8; i < 8 * kRouterCols; i += 256 * 8) {
    const int tt = i / kRouterCols, c = i % kRouterCols;
    *reinterpret_cast<uint4*>(&s_x[tt][c]) = (t0 + tt < T && c < hc) ? *reinterpret_cast<const uint4*>(x + (long long)(t0 + tt) * H + h0 + c)
                                                                    : make_uint4(0, 0, 0, 0);
  }
  __syncthreads();
  float* out = planes + (long long)blockIdx.z * T * E;
#pragma unroll 1
  for (int ee = 0; ee < 4; ee++) {
    const int e = blockIdx.y * 32 + warp * 4 + ee;
    if (e >= E) break;
    const float* wr = w + (long long)e * H + h0;
    float4 wv[8];
#pragma unroll
    for (int u = 0; u < 8; u++) {
      const int c = u * 128 + lane * 4;
      wv[u] = c < hc ? *reinterpret_cast<const float4*>(wr + c) : make_float4(0, 0, 0, 0);
    }
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
    for (int u = 0; u < 8; u++) {
#pragma unroll
      for (int tt = 0; tt < 8; tt++) {
        const uint2 xv = *reinterpret_cast<const uint2*>(&s_x[tt][u * 128 + lane * 4]);
        const float2 a = unpack_bf16x2(xv.x), b = unpack_bf16x2(xv.y);
        acc[tt] = fmaf(wv[u].x, a.x, fmaf(wv[u].y, a.y, fmaf(wv[u].z, b.x, fmaf(wv[u].w, b.y, acc[tt]))));
      }
    }
#pragma unroll
    for (int tt = 0; tt < 8; tt++) {
      const float v = warp_sum(acc[tt]);
      if (lane == 0 && t0 + tt < T) out[(long long)(t0 + tt) * E + e] = v;
    }
  }
}

// one CTA per token
__global__ void __launch_bounds__(256) moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ pos, const float* __restrict__ w,
                                                         const __nv_bfloat16* __restrict__ add_in, __nv_bfloat16* __restrict__ out, int top_k, int H) {
  pdl_wait(); pdl_trigger();      // dependent launch: nothing above this line touches global memory
  const int t = blockIdx.x;
  __shared__ int s_pos[64]; __shared__ float s_w[64];
  if (threadIdx.x < top_k) { s_pos[threadIdx.x] = pos[(long long)t * top_k + threadIdx.x]; s_w[threadIdx.x] = w[(long long)t * top_k + threadIdx.x]; }
  __syncthreads();
  // blockIdx.y splits the row into column slices: with one CTA per token a decode batch would occupy fewer CTAs than there
  // are SMs, each with 32 KB of loads in flight, a fraction of what it takes to keep HBM busy
  const int slice = (((H + 7) / 8 + gridDim.y - 1) / gridDim.y) * 8;
  const int c_end = min(H, ((int)blockIdx.y + 1) * slice);
  for (int c = blockIdx.y * slice + threadIdx.x * 8; c < c_end; c += blockDim.x * 8) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    // eight expert rows are fetched before any is used: the loads are independent and the kernel is latency-bound
    for (int k0 = 0; k0 < top_k; k0 += 8) {
      uint4 v[8];
#pragma unroll
      for (int q = 0; q < 8; q++) {
        const int r = k0 + q < top_k ? s_pos[k0 + q] : -1;
        v[q] = r >= 0 ? *reinterpret_cast<const uint4*>(y + (long long)r * H + c) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int q = 0; q < 8; q++) {
        const float wk = k0 + q < top_k ? s_w[k0 + q] : 0.f;
        const uint32_t u[4] = {v[q].x, v[q].y, v[q].z, v[q].w};
#pragma unroll
        for (int j = 0; j < 4; j++) { float2 f = unpack_bf16x2(u[j]); acc[2 * j] += wk * f.x; acc[2 * j + 1] += wk * f.y; }
      }
    }
    if (add_in) {
      // the routed sum is rounded to bf16 before the shared-expert output is added, as in the unfused form
      uint4 v = *reinterpret_cast<const uint4*>(add_in + (long long)t * H + c);
      uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; j++) {
        float2 f = unpack_bf16x2(u[j]); float2 r = unpack_bf16x2(pack_bf16x2(acc[2 * j], acc[2 * j + 1]));
        acc[2 * j] = r.x + f.x; acc[2 * j + 1] = r.y + f.y;
      }
    }
    *reinterpret_cast<uint4*>(out + (long long)t * H + c) =
        make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
  }
}

}  // namespace ne

using namespace ne;

// balance_ranks > 0: replace the chosen ids by ids dealt evenly over that many EP ranks (weights kept).  log2phy [E, max_rep] /
// logcnt [E] (device int32, optional): remap every logical id to one of its physical replicas.
extern "C" int ne_moe_route(const float* logits, const float* bias, int* idx, float* w, int T, int E, int top_k, int n_group,
                            int topk_group, int norm, float scale, int softmax, int planes, int balance_ranks, const int* log2phy,
                            const int* logcnt, int max_rep, cudaStream_t st) {
  if (T <= 0) return 0;
  if (E > kMaxExperts || top_k > 64 || n_group > 64 || (n_group > 1 && E % n_group) || planes < 1) return 1001;
  if (balance_ranks < 0 || (balance_ranks > 0 && E % balance_ranks) || (log2phy && (!logcnt || max_rep < 1))) return 1001;
  return (int)launch_pdl(moe_route_kernel, dim3((T + 3) / 4), dim3(128), 0, st, logits, bias, idx, w, T, E, top_k, n_group, topk_group, norm, scale, softmax,
                         planes, balance_ranks, log2phy, logcnt, max_rep);
}

// Outputs: counts [E_local], slot [T*K] (scratch), row_start [E_local+1], pos [T*K], and the
// expert-major activations (bf16, or e4m3 + scales with leading dimension s_ld >= max_rows).
extern "C" int ne_moe_dispatch_local(const void* x, const int* idx, int* counts, int* slot, int* row_start, int* pos, void* a_bf16,
                                     void* a_q, float* a_s, int s_ld, int T, int top_k, int H, int expert_offset, int E_local,
                                     int max_rows, int align, cudaStream_t st) {
  if (T <= 0) return 0;
  if (E_local > kMaxExperts || H % 128) return 1001;
  int n = T * top_k;
  if (top_k > 64) return 1001;
  cudaError_t e = launch_pdl(moe_count_scan_kernel, dim3(1), dim3(1024), 0, st, idx, counts, slot, row_start, n, expert_offset, E_local, align);
  if (e != cudaSuccess) return (int)e;
  return (int)launch_pdl(moe_scatter_kernel, dim3(T), dim3(256), (size_t)H + (H / 128) * 4, st, (const __nv_bfloat16*)x, idx, slot, row_start, pos,
                         (__nv_bfloat16*)a_bf16, (uint8_t*)a_q, a_s, s_ld, top_k, H, expert_offset, E_local, max_rows, g_scale_pow2);
}

extern "C" int ne_moe_combine_local(const void* y, const int* pos, const float* w, const void* add_in, void* out, int T, int top_k, int H,
                                    cudaStream_t st) {
  if (T <= 0) return 0;
  if (H % 8 || top_k > 64) return 1001;
  const int slices = T >= 2048 ? 1 : (T >= 512 ? 2 : 4);      // enough CTAs per SM at decode sizes, one pass over the tables per token otherwise
  return (int)launch_pdl(moe_combine_kernel, dim3(dim3(T, slices)), dim3(256), 0, st, (const __nv_bfloat16*)y, pos, w, (const __nv_bfloat16*)add_in, (__nv_bfloat16*)out, top_k, H);
}

// x bf16 [T, H], w fp32 [E, H] -> partial logits fp32 [ne_router_planes(H), T, E]; their sum over the first axis is x . w^T
extern "C" int ne_router_planes(int H) { return (H + kRouterCols - 1) / kRouterCols; }
extern "C" int ne_router_gemv(const void* x, const float* w, float* planes, int T, int E, int H, cudaStream_t st) {
  if (T <= 0) return 0;
  if (H % 128) return 1001;
  return (int)launch_pdl(router_gemv_kernel, dim3(dim3((T + 7) / 8, (E + 31) / 32, ne_router_planes(H))), dim3(256), 0, st, (const __nv_bfloat16*)x, w, planes, T, E, H);
}
