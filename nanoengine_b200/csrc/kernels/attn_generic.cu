// Shape-generic paged attention on CUDA cores: the path for head sizes the tensor-core kernels do not cover
// (small test models), for DSA sparse key lists, and for GQA caches.  One CTA per (query token, group of 4 heads),
// one warp per head; keys are staged through shared memory 32 at a time, each lane scores one key, the
// softmax is online, and each lane owns a slice of the output dimensions.
//
//   MLA:  q [T, H, Dk], cache rows [Dk] (first Dv values double as V), out [T, H, Dv]
//   GQA:  q [T, Hq, D], k/v caches [slots, Hkv, D], out [T, Hq, D]
// Keys of a query: positions [0, limit] of its sequence through the block table (causal), or an explicit list of
// physical slots (sparse, -1 = skip).  Cache dtype bf16 or e4m3 (query is then clamped and cast to e4m3 as well).
//
// Replaces in the reference: attention/base.py:451-525 (SDPA reference), flash_mla sparse decode call sites
// (layers/backends/mla/flash_mla.py:22-121) for the sparse case, flashinfer / FA paged GQA wrappers.
#include "ptx.cuh"

namespace ne {

constexpr int kKeysPerTile = 32;
constexpr int kHeadsPerCta = 4;

struct AttnArgs {
  const __nv_bfloat16* q; long long q_tok_stride; int q_head_stride;
  const void* k_cache; const void* v_cache;      // v_cache == nullptr: V is the first Dv values of the K row (MLA)
  long long kv_slot_stride; int kv_head_stride;   // in elements
  int kv_group;                                   // query heads per kv head (1 for MLA where kv_head_stride = 0)
  const int* block_tables; int bt_stride; int block_size;
  const int* cu_seqlens_q; const int* context_lens; int num_seqs;
  const int* sparse; int topk;                    // [T, topk] physical slots or nullptr
  __nv_bfloat16* out; long long o_tok_stride; int o_head_stride;
  float* lse;                                     // optional [T, H] natural-log LSE
  int T, H, Dk, Dv; float scale; int fp8;
  int window;                                     // > 0: a query sees only the last `window` key positions up to its own (sliding-window layers)
  int noncausal;                                  // 1: every query sees all keys of its sequence (vision encoder)
  int heads_per_cta;                              // 4, or 1 when every query head has its own kv head (the CTA stages one kv head)
};

__device__ __forceinline__ float load_kv(const void* base, long long idx, int fp8) {
  return fp8 ? e4m3_to_float(reinterpret_cast<const uint8_t*>(base)[idx]) : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
}

__global__ void __launch_bounds__(128) attn_generic_kernel(const AttnArgs a) {
  pdl_wait(); pdl_trigger();      // dependent launch: nothing above this line touches global memory
  extern __shared__ float sm[];
  // layout: q [4][Dk] | ktile [32][Dk+1] | vtile [32][Dv+1] (only when V is separate)
  const int Dk = a.Dk, Dv = a.Dv;
  float* sq = sm;
  float* sk = sq + kHeadsPerCta * Dk;
  float* sv = a.v_cache ? sk + kKeysPerTile * (Dk + 1) : nullptr;
  const int t = blockIdx.x, h0 = blockIdx.y * a.heads_per_cta;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = h0 + warp;
  const bool head_ok = h < a.H && warp < a.heads_per_cta;

  // which sequence owns token t
  int lo = 0, hi = a.num_seqs;
  while (lo + 1 < hi) { int mid = (lo + hi) >> 1; if (a.cu_seqlens_q[mid] <= t) lo = mid; else hi = mid; }
  const int seq = lo;
  const int q_len = a.cu_seqlens_q[seq + 1] - a.cu_seqlens_q[seq];
  const int ctx = a.context_lens[seq];
  const int limit = a.noncausal ? ctx - 1 : ctx - q_len + (t - a.cu_seqlens_q[seq]);   // last visible key position
  const int n_keys = a.sparse ? a.topk : limit + 1;
  const int first_key = (a.window > 0 && !a.sparse) ? max(0, limit - a.window + 1) : 0;

  for (int i = threadIdx.x; i < kHeadsPerCta * Dk; i += blockDim.x) {
    int hh = h0 + i / Dk, d = i % Dk;
    float v = (hh < a.H && i / Dk < a.heads_per_cta) ? __bfloat162float(a.q[(long long)t * a.q_tok_stride + (long long)hh * a.q_head_stride + d]) : 0.f;
    if (a.fp8) v = e4m3_to_float(to_e4m3(fminf(fmaxf(v, -448.f), 448.f)));
    sq[i] = v;
  }
  // all 4 heads of a CTA must read the same kv head: heads per CTA divide the group size, or the group size is 1 with stride 0
  const int kvh = (a.kv_group > 0) ? h0 / a.kv_group : 0;
  const int per_lane = (Dv + 31) / 32;
  float acc[20];
#pragma unroll
  for (int j = 0; j < 20; j++) acc[j] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;
  const float c = a.scale * 1.4426950408889634f;
  const int* bt = a.block_tables + (long long)seq * a.bt_stride;

  for (int k0 = first_key / kKeysPerTile * kKeysPerTile; k0 < n_keys; k0 += kKeysPerTile) {
    __syncthreads();
    // stage 32 key rows (and value rows) as fp32
    for (int r = warp; r < kKeysPerTile; r += 4) {
      int kidx = k0 + r;
      long long slot = -1;
      if (kidx < n_keys) {
        if (a.sparse) slot = a.sparse[(long long)t * a.topk + kidx];
        else {
          const int page = bt[kidx / a.block_size];
          slot = (a.block_size == 1 || NE_INDEX_OK(page, BK_CACHE_PAGES, 23, __LINE__)) ? (long long)page * a.block_size + kidx % a.block_size : -1;
        }
      }
      for (int d = lane; d < Dk; d += 32)
        sk[r * (Dk + 1) + d] = slot >= 0 ? load_kv(a.k_cache, slot * a.kv_slot_stride + (long long)kvh * a.kv_head_stride + d, a.fp8) : 0.f;
      if (sv) for (int d = lane; d < Dv; d += 32)
        sv[r * (Dv + 1) + d] = slot >= 0 ? load_kv(a.v_cache, slot * a.kv_slot_stride + (long long)kvh * a.kv_head_stride + d, a.fp8) : 0.f;
      if (lane == 0) sk[r * (Dk + 1) + Dk] = slot >= 0 ? 1.f : 0.f;   // validity marker in the padding column
    }
    __syncthreads();
    if (!head_ok) continue;
    // lane scores key `lane`
    const float* kr = sk + lane * (Dk + 1);
    const float* qr = sq + warp * Dk;
    float s = 0.f;
    for (int d = 0; d < Dk; d++) s = fmaf(qr[d], kr[d], s);
    bool valid = (k0 + lane < n_keys) && (k0 + lane >= first_key) && kr[Dk] != 0.f;
    float tl = valid ? s * c : -INFINITY;
    float m_new = fmaxf(m_run, warp_max(tl));
    if (m_new == -INFINITY) continue;
    float alpha = exp2f(m_run - m_new);
    float p = valid ? exp2f(tl - m_new) : 0.f;
    l_run = l_run * alpha + warp_sum(p);
    m_run = m_new;
    const float* vt = sv ? sv : sk;
    const int vstride = sv ? Dv + 1 : Dk + 1;
#pragma unroll
    for (int j = 0; j < 20; j++) acc[j] *= alpha;
    for (int kk = 0; kk < kKeysPerTile; kk++) {
      float pk = __shfl_sync(0xffffffffu, p, kk);
      if (pk == 0.f) continue;
#pragma unroll
      for (int j = 0; j < 20; j++) {
        int d = lane + 32 * j;
        if (j < per_lane && d < Dv) acc[j] = fmaf(pk, vt[kk * vstride + d], acc[j]);
      }
    }
  }
  if (!head_ok) return;
  float inv = l_run > 0.f ? 1.f / l_run : 0.f;
#pragma unroll
  for (int j = 0; j < 20; j++) {
    int d = lane + 32 * j;
    if (j < per_lane && d < Dv) a.out[(long long)t * a.o_tok_stride + (long long)h * a.o_head_stride + d] = __float2bfloat16(acc[j] * inv);
  }
  if (a.lse && lane == 0) a.lse[(long long)t * a.H + h] = l_run > 0.f ? (m_run * 0.6931471805599453f + logf(l_run)) : -INFINITY;
}

// out = sum_s softmax_s(lse) * part_s  for split-KV attention.  part [S, rows, D] fp32 (already normalised), lse2 [S, rows] (log2 domain).
__global__ void attn_merge_kernel(const float* __restrict__ part, const float* __restrict__ lse2, __nv_bfloat16* __restrict__ out,
                                  int splits, long long rows, int D, int out_row_stride) {
  pdl_wait(); pdl_trigger();      // dependent launch: nothing above this line touches global memory
  long long row = blockIdx.x;
  float m = -INFINITY;
  for (int s = 0; s < splits; s++) m = fmaxf(m, lse2[(long long)s * rows + row]);
  float den = 0.f;
  for (int s = 0; s < splits; s++) { float l = lse2[(long long)s * rows + row]; den += (l == -INFINITY) ? 0.f : exp2f(l - m); }
  float inv = den > 0.f ? 1.f / den : 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < splits; s++) {
      float l = lse2[(long long)s * rows + row];
      if (l != -INFINITY) acc += exp2f(l - m) * part[((long long)s * rows + row) * D + d];
    }
    out[row * out_row_stride + d] = __float2bfloat16(acc * inv);
  }
}

// ---- sampling --------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t hash32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16; return x;
}

// One CTA per row.  temperature < 1e-5: argmax.  Otherwise Gumbel-max: argmax(logit / T + g), g = -log(-log(u)), u from a
// counter-based hash of (seed, row, column).  Optionally the log-probability of the chosen token under softmax(logits).
__global__ void __launch_bounds__(1024) sample_kernel(const float* __restrict__ logits, const float* __restrict__ temps, long long* __restrict__ tok,
                                                     float* __restrict__ logprob, int V, uint64_t seed) {
  pdl_wait(); pdl_trigger();      // dependent launch: nothing above this line touches global memory
  __shared__ float s_val[32]; __shared__ int s_idx[32]; __shared__ float s_m[32]; __shared__ float s_s[32];
  const int row = blockIdx.x;
  const float* lr = logits + (long long)row * V;
  const float temp = temps[row];
  const bool greedy = temp < 1e-5f;
  const float it = greedy ? 1.f : 1.f / temp;
  float best = -INFINITY; int bi = 0x7fffffff; float m = -INFINITY, ssum = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    float x = lr[i];
    float v = x * it;
    if (!greedy) {
      uint32_t hsh = hash32((uint32_t)i * 0x9e3779b9u ^ hash32((uint32_t)row ^ hash32((uint32_t)seed ^ (uint32_t)(seed >> 32))));
      float u = fmaxf((float)(hsh >> 8) * (1.0f / 16777216.0f), 1e-20f);
      v += -__logf(-__logf(u));
    }
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    if (logprob) { float nm = fmaxf(m, x); ssum = ssum * __expf(m - nm) + __expf(x - nm); m = nm; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ob = __shfl_xor_sync(0xffffffffu, best, o); int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, ssum, o);
    float nm = fmaxf(m, om);
    ssum = (nm == -INFINITY) ? 0.f : ssum * __expf(m - nm) + os * __expf(om - nm); m = nm;
  }
  if (lane == 0) { s_val[warp] = best; s_idx[warp] = bi; s_m[warp] = m; s_s[warp] = ssum; }
  __syncthreads();
  if (warp == 0) {
    best = lane < nw ? s_val[lane] : -INFINITY; bi = lane < nw ? s_idx[lane] : 0x7fffffff;
    m = lane < nw ? s_m[lane] : -INFINITY; ssum = lane < nw ? s_s[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ob = __shfl_xor_sync(0xffffffffu, best, o); int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
      float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, ssum, o);
      float nm = fmaxf(m, om);
      ssum = (nm == -INFINITY) ? 0.f : ssum * __expf(m - nm) + os * __expf(om - nm); m = nm;
    }
    if (lane == 0) {
      tok[row] = bi;
      if (logprob) logprob[row] = lr[bi] - (m + __logf(ssum));
    }
  }
}

}  // namespace ne

using namespace ne;

extern "C" int ne_attn_generic(const void* q, long long q_tok_stride, int q_head_stride, const void* k_cache, const void* v_cache,
                               long long kv_slot_stride, int kv_head_stride, int kv_group, const int* block_tables, int bt_stride,
                               int block_size, const int* cu_seqlens_q, const int* context_lens, int num_seqs, const int* sparse, int topk,
                               void* out, long long o_tok_stride, int o_head_stride, float* lse, int T, int H, int Dk, int Dv, float scale,
                               int fp8, int window, int noncausal, cudaStream_t st) {
  if (T <= 0) return 0;
  if (Dv > 640 || (kv_group > 1 && kv_group % kHeadsPerCta != 0)) return 1001;
  AttnArgs a;
  a.q = (const __nv_bfloat16*)q; a.q_tok_stride = q_tok_stride; a.q_head_stride = q_head_stride; a.k_cache = k_cache; a.v_cache = v_cache;
  a.kv_slot_stride = kv_slot_stride; a.kv_head_stride = kv_head_stride; a.kv_group = kv_group; a.block_tables = block_tables;
  a.bt_stride = bt_stride; a.block_size = block_size; a.cu_seqlens_q = cu_seqlens_q; a.context_lens = context_lens; a.num_seqs = num_seqs;
  a.sparse = sparse; a.topk = topk; a.out = (__nv_bfloat16*)out; a.o_tok_stride = o_tok_stride; a.o_head_stride = o_head_stride; a.lse = lse;
  a.T = T; a.H = H; a.Dk = Dk; a.Dv = Dv; a.scale = scale; a.fp8 = fp8; a.window = window; a.noncausal = noncausal;
  // multi-head attention proper (one kv head per query head, separate V): the four query heads of a CTA would need four
  // different key tiles, so a CTA serves one head there
  a.heads_per_cta = (kv_group == 1 && kv_head_stride != 0 && v_cache != nullptr) ? 1 : kHeadsPerCta;
  size_t smem = sizeof(float) * ((size_t)kHeadsPerCta * Dk + (size_t)kKeysPerTile * (Dk + 1) + (v_cache ? (size_t)kKeysPerTile * (Dv + 1) : 0));
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_generic_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  dim3 grid(T, (H + a.heads_per_cta - 1) / a.heads_per_cta);
  return (int)launch_pdl(attn_generic_kernel, dim3(grid), dim3(128), smem, st, a);
}

extern "C" int ne_attn_merge(const float* part, const float* lse2, void* out, int splits, long long rows, int D, int out_row_stride, cudaStream_t st) {
  if (rows <= 0) return 0;
  return (int)launch_pdl(attn_merge_kernel, dim3((unsigned)rows), dim3(128), 0, st, part, lse2, (__nv_bfloat16*)out, splits, rows, D, out_row_stride);
}

extern "C" int ne_sample(const float* logits, const float* temps, long long* tok, float* logprob, int rows, int V, unsigned long long seed,
                         cudaStream_t st) {
  if (rows <= 0) return 0;
  return (int)launch_pdl(sample_kernel, dim3(rows), dim3(1024), 0, st, logits, temps, tok, logprob, V, (uint64_t)seed);
}
