// Device-side verification of MTP (multi-token prediction) drafts.
//
// A verify pass runs the target model over rows [last token, d1 .. dN] of every sequence and yields logits [B, N+1, V].
// Two kernels turn them into the step's result without a host round trip:
//
//   mtp_row_stats   one CTA per row: arg-max, log-sum-exp of the row at the sequence's temperature and the scaled logit of
//                   the draft token that row has to confirm (row i confirms d_{i+1})
//   mtp_finalize    one CTA per sequence: accepted count = longest prefix of confirmed drafts - greedy rows confirm by
//                   arg-max equality, sampled rows by one uniform coin per position against p_target(draft) - then the next
//                   token: the arg-max of the stop row (greedy) or a Gumbel-max sample of the stop row with the rejected
//                   draft masked out (unmasked when every draft was accepted), which preserves the target distribution.
//                   Writes the emitted bundle [accepted drafts, next token], the token inputs of the predictor's
//                   draft-extend pass, and the log-probability of the next token under the unmasked target row.
//
// Replaces in the reference: runtime/runner/mtp_runner.py:111-187 (linear_rejection_sample), :190-208 (linear_greedy_verify)
// and the host-side bookkeeping of lazy_verify_sample :536-624, which run as PyTorch ops with host synchronisation.
#include "ptx.cuh"

namespace ne {

__device__ __forceinline__ uint32_t mtp_hash32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16; return x;
}
__device__ __forceinline__ float mtp_uniform(uint64_t seed, uint32_t a, uint32_t b) {
  const uint32_t h = mtp_hash32(b * 0x9e3779b9u ^ mtp_hash32(a ^ mtp_hash32((uint32_t)seed ^ (uint32_t)(seed >> 32))));
  return fmaxf((float)(h >> 8) * (1.0f / 16777216.0f), 1e-20f);
}

struct RowStat { int argmax; float lse; float v_draft; int pad; };

// block-wide reduction of (best value, its lowest index) and of an online (max, sum-exp) pair
struct ArgMaxLse { float best; int bi; float m; float s; };
__device__ __forceinline__ ArgMaxLse combine(ArgMaxLse a, const ArgMaxLse& b) {
  if (b.best > a.best || (b.best == a.best && b.bi < a.bi)) { a.best = b.best; a.bi = b.bi; }
  const float nm = fmaxf(a.m, b.m);
  a.s = (nm == -INFINITY) ? 0.f : a.s * __expf(a.m - nm) + b.s * __expf(b.m - nm);
  a.m = nm;
  return a;
}
__device__ __forceinline__ ArgMaxLse block_reduce(ArgMaxLse v, ArgMaxLse* smem) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMaxLse t;
    t.best = __shfl_xor_sync(0xffffffffu, v.best, o); t.bi = __shfl_xor_sync(0xffffffffu, v.bi, o);
    t.m = __shfl_xor_sync(0xffffffffu, v.m, o); t.s = __shfl_xor_sync(0xffffffffu, v.s, o);
    v = combine(v, t);
  }
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  if (warp == 0) {
    v = lane < nw ? smem[lane] : ArgMaxLse{-INFINITY, 0x7fffffff, -INFINITY, 0.f};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgMaxLse t;
      t.best = __shfl_xor_sync(0xffffffffu, v.best, o); t.bi = __shfl_xor_sync(0xffffffffu, v.bi, o);
      t.m = __shfl_xor_sync(0xffffffffu, v.m, o); t.s = __shfl_xor_sync(0xffffffffu, v.s, o);
      v = combine(v, t);
    }
    if (lane == 0) smem[0] = v;
  }
  __syncthreads();
  v = smem[0];
  __syncthreads();
  return v;
}

__global__ void __launch_bounds__(1024) mtp_row_stats_kernel(const float* __restrict__ logits, const long long* __restrict__ drafts,
                                                            const float* __restrict__ temps, RowStat* __restrict__ stats, int N, int V) {
  pdl_wait(); pdl_trigger();
  __shared__ ArgMaxLse s_red[32];
  const int row = blockIdx.x, b = row / (N + 1), i = row - b * (N + 1);
  const float* lr = logits + (long long)row * V;
  const float temp = temps[b];
  const float it = temp < 1e-5f ? 1.f : 1.f / temp;
  ArgMaxLse v{-INFINITY, 0x7fffffff, -INFINITY, 0.f};
  for (int c = threadIdx.x; c < V; c += blockDim.x) {
    const float x = lr[c] * it;
    if (x > v.best || (x == v.best && c < v.bi)) { v.best = x; v.bi = c; }
    const float nm = fmaxf(v.m, x);
    v.s = v.s * __expf(v.m - nm) + __expf(x - nm); v.m = nm;
  }
  v = block_reduce(v, s_red);
  if (threadIdx.x == 0) {
    RowStat st;
    st.argmax = v.bi; st.lse = v.m + __logf(v.s); st.pad = 0;
    long long d = i < N ? drafts[(long long)b * N + i] : -1;
    st.v_draft = (d >= 0 && d < V) ? lr[d] * it : -INFINITY;
    stats[row] = st;
  }
}

__global__ void __launch_bounds__(1024) mtp_finalize_kernel(const float* __restrict__ logits, const long long* __restrict__ drafts,
                                                           const float* __restrict__ temps, const int* __restrict__ have,
                                                           const RowStat* __restrict__ stats, const float* __restrict__ coins,
                                                           int* __restrict__ num_accepted, long long* __restrict__ next_token,
                                                           long long* __restrict__ bundle, long long* __restrict__ extend_tokens,
                                                           float* __restrict__ logprob, int N, int V, int force_accept, uint64_t seed,
                                                           const unsigned long long* __restrict__ seed_ptr) {
  pdl_wait(); pdl_trigger();
  __shared__ ArgMaxLse s_red[32];
  __shared__ int s_acc;
  if (seed_ptr) seed = *seed_ptr;        // a counter in device memory: a replayed CUDA graph draws fresh noise every step
  const int b = blockIdx.x;
  const float temp = temps[b];
  const bool greedy = temp < 1e-5f;
  const float it = greedy ? 1.f : 1.f / temp;
  const RowStat* st = stats + (long long)b * (N + 1);
  const long long* dr = drafts + (long long)b * N;
  if (threadIdx.x == 0) {
    int acc = 0;
    if (force_accept >= 0) acc = force_accept < N ? force_accept : N;
    else if (!have || have[b]) {
      for (; acc < N; acc++) {
        bool ok;
        if (greedy) ok = (long long)st[acc].argmax == dr[acc];
        else {
          const float u = coins ? coins[(long long)b * N + acc] : mtp_uniform(seed, 0x51ed27u + (uint32_t)b, (uint32_t)acc);
          ok = u < __expf(st[acc].v_draft - st[acc].lse);
        }
        if (!ok) break;
      }
    }
    s_acc = acc;
  }
  __syncthreads();
  const int acc = s_acc;
  const float* lr = logits + ((long long)b * (N + 1) + acc) * V;
  long long nxt;
  if (greedy || force_accept >= 0) {
    nxt = st[acc].argmax;
  } else {
    // Gumbel-max over the stop row; the rejected draft cannot be drawn again
    const long long masked = (acc < N && (!have || have[b])) ? dr[acc] : -1;
    ArgMaxLse v{-INFINITY, 0x7fffffff, -INFINITY, 0.f};
    for (int c = threadIdx.x; c < V; c += blockDim.x) {
      if (c == masked) continue;
      const float g = -__logf(-__logf(mtp_uniform(seed, 0xa511e9b3u ^ (uint32_t)b, (uint32_t)c)));
      const float x = lr[c] * it + g;
      if (x > v.best || (x == v.best && c < v.bi)) { v.best = x; v.bi = c; }
    }
    v = block_reduce(v, s_red);
    nxt = v.bi;
  }
  if (threadIdx.x == 0) {
    num_accepted[b] = acc;
    next_token[b] = nxt;
    if (logprob) logprob[b] = lr[nxt] * it - st[acc].lse;
  }
  // the emitted bundle (accepted drafts, then the next token, -1 beyond) and the predictor's inputs for the draft-extend pass
  // (row i pairs token i+1 with hidden state i; rows past the accepted prefix repeat the next token and are never read)
  for (int i = threadIdx.x; i <= N; i += blockDim.x) {
    if (bundle) bundle[(long long)b * (N + 1) + i] = i < acc ? dr[i] : (i == acc ? nxt : -1);
    if (extend_tokens) extend_tokens[(long long)b * (N + 1) + i] = i < acc ? dr[i] : nxt;
  }
}

// Metadata of chain step k (k = 1 .. N-1) of the draft predictor, built on the device from the accepted counts so the chain needs
// no host round trip: the token drafted at step k sits at position base_len[b] + acc[b] + k - 1.
__global__ void mtp_chain_meta_kernel(const int* __restrict__ base_len, const int* __restrict__ num_accepted, const int* __restrict__ block_tables,
                                      int bt_stride, int block_size, int k, int B, long long* __restrict__ positions,
                                      long long* __restrict__ slot_mapping, int* __restrict__ context_lens) {
  pdl_wait(); pdl_trigger();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const int pos = base_len[b] + num_accepted[b] + k - 1;
  positions[b] = pos;
  context_lens[b] = pos + 1;
  slot_mapping[b] = (long long)block_tables[(long long)b * bt_stride + pos / block_size] * block_size + pos % block_size;
}

}  // namespace ne

using namespace ne;

// logits fp32 [B, N+1, V]; drafts int64 [B, N]; temps fp32 [B]; have int32 [B] or null (0 = the sequence has no drafts: accept
// none); coins fp32 [B, N] or null (uniforms for the acceptance test; null = drawn from `seed`); stats: scratch of
// B * (N+1) * 16 bytes.  Outputs: num_accepted int32 [B], next_token int64 [B], bundle int64 [B, N+1] or null, extend_tokens
// int64 [B, N+1] or null, logprob fp32 [B] or null.  force_accept >= 0 pins the accepted count (benchmarks).  seed_ptr (device,
// optional) overrides `seed` with a value read at run time.
extern "C" int ne_mtp_verify(const float* logits, const long long* drafts, const float* temps, const int* have, const float* coins, void* stats,
                             int* num_accepted, long long* next_token, long long* bundle, long long* extend_tokens, float* logprob, int B,
                             int N, int V, int force_accept, unsigned long long seed, const unsigned long long* seed_ptr, cudaStream_t st) {
  if (B <= 0) return 0;
  if (N < 0 || V < 1) return 1001;
  cudaError_t e = launch_pdl(mtp_row_stats_kernel, dim3(B * (N + 1)), dim3(1024), 0, st, logits, drafts, temps, (RowStat*)stats, N, V);
  if (e != cudaSuccess) return (int)e;
  return (int)launch_pdl(mtp_finalize_kernel, dim3(B), dim3(1024), 0, st, logits, drafts, temps, have, (const RowStat*)stats, coins, num_accepted,
                         next_token, bundle, extend_tokens, logprob, N, V, force_accept, (uint64_t)seed, seed_ptr);
}

extern "C" int ne_mtp_chain_meta(const int* base_len, const int* num_accepted, const int* block_tables, int bt_stride, int block_size, int k, int B,
                                 long long* positions, long long* slot_mapping, int* context_lens, cudaStream_t st) {
  if (B <= 0) return 0;
  return (int)launch_pdl(mtp_chain_meta_kernel, dim3((B + 127) / 128), dim3(128), 0, st, base_len, num_accepted, block_tables, bt_stride, block_size, k,
                         B, positions, slot_mapping, context_lens);
}
