// DSA lightning indexer: query / key preparation, fp8 logits on the tensor cores, radix top-k with page translation.
//
//   indexer_prep    one warp per 128-wide row: [LayerNorm] -> RoPE on the first `rope` dims (pairs (i, i + rope/2)) ->
//                   128-point Hadamard -> one power-of-two scale per row -> e4m3; keys go straight into their cache page
//                   (page = [bs x 128 B keys | bs x fp32 scales]), queries into a dense [rows, 128] buffer + scales.
//   indexer_logits  logits[t, j] = k_scale[j] * sum_h w[t, h] * relu(q8[t, h, :] . k8[j, :]) for the keys j the token may see.
//                   One CTA per (token, key split): Q (heads x 128 B) stays in shared memory, key tiles of 128 keys (two pages)
//                   stream through a TMA ring, S^T = K Q^T is one group of four tcgen05 MMAs (M = 128 keys, N = 64 heads,
//                   K = 32) into a double-buffered TMEM accumulator.  Keys are the accumulator's rows, so each of the 128
//                   epilogue threads owns one key, reads its 64 head scores from TMEM and folds relu, head weight and the
//                   head sum in registers: no cross-lane reduction.
//   indexer_topk    per token: 3-pass radix select (11 + 11 + 10 bits) of the k largest logits among the visible keys, written
//                   as physical slot ids (block_table[idx / bs] * bs + idx % bs), -1 padded.
//
// Replaces in the reference: deep_gemm.fp8_mqa_logits / fp8_paged_mqa_logits (layers/backends/dsa/indexer/lightning.py:
// 1081-1492), kernel/jit/sgl/csrc/deepseek_v4/{indexer_q.cuh, topk.cuh, topk_v2.cuh}, fast-hadamard-transform/hadamard_jit.cuh
// and the Triton key path (triton/generic/indexer_transform.py, fp8_ue8m0_quant.py:370).
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <math.h>

#include "ptx.cuh"
#include "tma_host.h"

namespace ne {

constexpr int kKernelIdx = 6;
constexpr int kIdxD = 128;                 // index head dim: one 128-byte swizzle row of e4m3
constexpr int kIdxPage = 64;               // keys per cache page
constexpr int kIdxTile = 128;              // keys per MMA tile (two pages)
constexpr int kIdxStages = 4;
constexpr int kIdxQBytes = 128 * 128;      // Q tile slot (only the first `heads` rows are fetched)
constexpr int kIdxKBytes = kIdxTile * 128;
constexpr int kIdxSmem = kIdxQBytes + kIdxStages * kIdxKBytes + 1024 + 256 + 64 * 4;
constexpr int kIdxThreads = 192;

// ---------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16(x)); }

// x: rows of 128 bf16 (row r at x + r * x_ld).  heads = rows per token (positions / slots are per token).
__global__ void __launch_bounds__(256) indexer_prep_kernel(const __nv_bfloat16* __restrict__ x, long long x_ld, int rows, int heads,
                                                          const __nv_bfloat16* __restrict__ ln_w, const __nv_bfloat16* __restrict__ ln_b, float eps,
                                                          const long long* __restrict__ positions, const float* __restrict__ rope_cache, int rope,
                                                          uint8_t* __restrict__ q_out, float* __restrict__ s_out,
                                                          uint8_t* __restrict__ cache, const long long* __restrict__ slots, int bs, long long page_bytes) {
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= rows) return;
  const int t = r / heads;
  const uint2 raw = *reinterpret_cast<const uint2*>(x + (long long)r * x_ld + lane * 4);
  const float2 p0 = unpack_bf16x2(raw.x), p1 = unpack_bf16x2(raw.y);
  float v[4] = {p0.x, p0.y, p1.x, p1.y};
  if (ln_w) {
    float s = warp_sum(v[0] + v[1] + v[2] + v[3]);
    const float mean = s * (1.f / kIdxD);
    float q = 0.f;
#pragma unroll
    for (int j = 0; j < 4; j++) q += (v[j] - mean) * (v[j] - mean);
    const float inv = rsqrtf(warp_sum(q) * (1.f / kIdxD) + eps);
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int e = lane * 4 + j;
      v[j] = bf16_round((v[j] - mean) * inv * __bfloat162float(ln_w[e]) + (ln_b ? __bfloat162float(ln_b[e]) : 0.f));
    }
  }
  // RoPE on elements [0, rope): pairs (i, i + rope/2).  With rope = 64 the partner of lane l (l < 16) is lane l ^ 8.
  {
    const int half = rope / 2, hl = half / 4;                 // lanes per half
    const float* cs = rope_cache + positions[t] * rope;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const float other = __shfl_xor_sync(0xffffffffu, v[j], hl);
      const int e = lane * 4 + j;
      if (e < rope) {
        const int i = e % half;
        const float c = cs[i], sn = cs[half + i];
        v[j] = bf16_round(e < half ? v[j] * c - other * sn : v[j] * c + other * sn);
      }
    }
  }
  // 128-point Walsh-Hadamard (Sylvester order): strides 1, 2 inside the lane, 4 .. 64 across lanes
  {
    float a0 = v[0] + v[1], a1 = v[0] - v[1], a2 = v[2] + v[3], a3 = v[2] - v[3];
    v[0] = a0 + a2; v[1] = a1 + a3; v[2] = a0 - a2; v[3] = a1 - a3;
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const float o = __shfl_xor_sync(0xffffffffu, v[j], m);
        v[j] = (lane & m) ? o - v[j] : v[j] + o;
      }
    }
    const float nrm = 0.08838834764831845f;                   // 128^-1/2
#pragma unroll
    for (int j = 0; j < 4; j++) v[j] = bf16_round(v[j] * nrm);
  }
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
  amax = fmaxf(warp_max(amax), 1e-4f);
  const float sc = exp2f(ceilf(log2f(amax / 448.f)));
  const float is = 1.f / sc;
  const uint32_t packed = pack_e4m3x4(v[0] * is, v[1] * is, v[2] * is, v[3] * is);
  if (cache) {
    const long long slot = slots[t];
    if (slot >= 0 && !NE_INDEX_OK(slot, BK_CACHE_ROWS, 22, __LINE__)) return;
    if (slot < 0) return;
    uint8_t* page = cache + (slot / bs) * page_bytes;
    const int off = (int)(slot % bs);
    *reinterpret_cast<uint32_t*>(page + (long long)off * kIdxD + lane * 4) = packed;
    if (lane == 0) *reinterpret_cast<float*>(page + (long long)bs * kIdxD + off * 4) = sc;
  } else {
    *reinterpret_cast<uint32_t*>(q_out + (long long)r * kIdxD + lane * 4) = packed;
    if (lane == 0) s_out[r] = sc;
  }
}

// ---------------------------------------------------------------------------------------------------------------------
struct IdxArgs {
  const float* head_w; const float* q_scale;        // [T, heads] each
  const uint8_t* cache; long long page_bytes;       // indexer cache, for the key scales
  const int* block_tables; int bt_stride;
  const int* cu_seqlens_q; const int* context_lens; int num_seqs;
  int T, heads, splits;
  float* logits; long long ld;                      // [T, ld] fp32
};

__global__ void __launch_bounds__(kIdxThreads, 1)
indexer_logits_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk, const IdxArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + kIdxQBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sK + kIdxStages * kIdxKBytes);
  // q_full | k_full[4] | k_empty[4] | s_full[2] | s_empty[2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* s_rw = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + 256);          // [64] head weight x query scale
  const uint32_t b_qfull = smem_u32(bars), b_kfull = smem_u32(bars + 1), b_kempty = smem_u32(bars + 5);
  const uint32_t b_sfull = smem_u32(bars + 9), b_sempty = smem_u32(bars + 11);
  const int warp = threadIdx.x >> 5;
  const int t = blockIdx.x, split = blockIdx.y;

  int lo = 0, hi = a.num_seqs;
  while (lo + 1 < hi) { int mid = (lo + hi) >> 1; if (a.cu_seqlens_q[mid] <= t) lo = mid; else hi = mid; }
  const int seq = lo;
  const int q_len = a.cu_seqlens_q[seq + 1] - a.cu_seqlens_q[seq];
  const int limit = a.context_lens[seq] - q_len + (t - a.cu_seqlens_q[seq]);     // last visible key position
  const int total_tiles = limit >= 0 ? limit / kIdxTile + 1 : 0;
  const int per_split = (total_tiles + a.splits - 1) / a.splits;
  const int tile_begin = split * per_split;
  const int n_tiles = max(0, min(total_tiles, tile_begin + per_split) - tile_begin);
  const int* bt = a.block_tables + (long long)seq * a.bt_stride;

  if (threadIdx.x == 0) {
    mbar_init(b_qfull, 1);
    for (int i = 0; i < kIdxStages; i++) { mbar_init(b_kfull + 8 * i, 1); mbar_init(b_kempty + 8 * i, 1); }
    for (int i = 0; i < 2; i++) { mbar_init(b_sfull + 8 * i, 1); mbar_init(b_sempty + 8 * i, 4); }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tq); tma_prefetch_desc(&tk);
  }
  if (threadIdx.x < 64) s_rw[threadIdx.x] = (int)threadIdx.x < a.heads ? a.head_w[(long long)t * a.heads + threadIdx.x] * a.q_scale[(long long)t * a.heads + threadIdx.x] : 0.f;
  if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), 128); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (n_tiles > 0 && elect_one()) {
      mbar_expect_tx(b_qfull, 64 * 128);
      tma_load_2d(smem_u32(sQ), &tq, b_qfull, 0, t * a.heads);
      for (int i = 0; i < n_tiles; i++) {
        const int s = i % kIdxStages;
        if (!mbar_wait(b_kempty + 8 * s, ((i / kIdxStages) & 1) ^ 1, abort_flag, kKernelIdx, 100 + s)) break;
        const int pg = (tile_begin + i) * 2;                       // first of the tile's two pages
        const bool two = (long long)(pg + 1) * kIdxPage <= limit;  // the second page holds at least one visible key
        mbar_expect_tx(b_kfull + 8 * s, two ? kIdxKBytes : kIdxKBytes / 2);
        tma_load_3d(smem_u32(sK + s * kIdxKBytes), &tk, b_kfull + 8 * s, 0, 0, bt[pg]);
        if (two) tma_load_3d(smem_u32(sK + s * kIdxKBytes + kIdxKBytes / 2), &tk, b_kfull + 8 * s, 0, 0, bt[pg + 1]);
      }
    }
  } else if (warp == 1) {
    if (n_tiles > 0 && elect_one()) {
      constexpr uint32_t kIdesc = make_idesc(FMT_E4M3, FMT_E4M3, 128, 64);        // M = 128 keys, N = 64 heads
      bool ok = mbar_wait(b_qfull, 0, abort_flag, kKernelIdx, 200);
      // the next tile's barriers are tested before this tile's MMAs are issued (a test costs ~150 cycles even when the phase
      // completed long ago; the blocking MMA issue hides it)
      bool pre_se = true, pre_k = mbar_test(b_kfull, 0);
      for (int i = 0; ok && i < n_tiles; i++) {
        const int sb = i & 1, s = i % kIdxStages;
        if (!pre_se && !mbar_wait(b_sempty + 8 * sb, ((i >> 1) & 1) ^ 1, abort_flag, kKernelIdx, 210 + sb)) break;
        if (!pre_k && !mbar_wait(b_kfull + 8 * s, (i / kIdxStages) & 1, abort_flag, kKernelIdx, 220 + s)) break;
        mbar_test2(b_sempty + 8 * ((i + 1) & 1), (((i + 1) >> 1) & 1) ^ 1, b_kfull + 8 * ((i + 1) % kIdxStages), ((i + 1) / kIdxStages) & 1,
                   pre_se, pre_k);
        tc_fence_after();
        const uint32_t qa = smem_u32(sQ), ka = smem_u32(sK + s * kIdxKBytes);
#pragma unroll
        for (int ks = 0; ks < 4; ks++) {
          uint64_t adesc = make_smem_desc(ka + ks * 32, 16, 1024, SW_128B);
          uint64_t bdesc = make_smem_desc(qa + ks * 32, 16, 1024, SW_128B);
          umma_f8(tmem_base + sb * 64, adesc, bdesc, kIdesc, ks != 0);
        }
        tc_commit(b_kempty + 8 * s);
        tc_commit(b_sfull + 8 * sb);
      }
    }
  } else {
    // thread = key: TMEM lane quadrant (warp % 4) x lane
    const int wq = warp & 3, lane = (int)lane_id();
    const int krow = wq * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(wq * 32) << 16;
    float rw[64];
#pragma unroll
    for (int h = 0; h < 64; h++) rw[h] = s_rw[h];
    float* out_row = a.logits + (long long)t * a.ld;
    bool s_ready = false;
    for (int i = 0; i < n_tiles; i++) {
      const int sb = i & 1;
      if (!s_ready && !mbar_wait(b_sfull + 8 * sb, (i >> 1) & 1, abort_flag, kKernelIdx, 300 + sb)) break;
      tc_fence_after();
      uint32_t r0[32], r1[32];
      tmem_ld_32x32b_x32(tmem_base + lane_addr + sb * 64, r0);
      tmem_ld_32x32b_x32(tmem_base + lane_addr + sb * 64 + 32, r1);
      s_ready = mbar_test(b_sfull + 8 * ((i + 1) & 1), ((i + 1) >> 1) & 1);      // answer wanted at the next loop top
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(b_sempty + 8 * sb);
      float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
      for (int h = 0; h < 32; h++) {
        acc0 = fmaf(fmaxf(__uint_as_float(r0[h]), 0.f), rw[h], acc0);
        acc1 = fmaf(fmaxf(__uint_as_float(r1[h]), 0.f), rw[32 + h], acc1);
      }
      const int key = (tile_begin + i) * kIdxTile + krow;
      if (key < a.ld) {
        float res = -INFINITY;
        if (key <= limit)
          res = (acc0 + acc1) * *reinterpret_cast<const float*>(a.cache + (long long)bt[key / kIdxPage] * a.page_bytes + kIdxPage * kIdxD + (key % kIdxPage) * 4);
        out_row[key] = res;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) for (int i = 0; i < 2000; i++) __nanosleep(1000);
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 128); }
}

// ---------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t float_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);          // larger float <=> larger key
}

__device__ __forceinline__ int ld_dsmem_i32(uint32_t addr) {
  int v;
  asm volatile("ld.shared::cluster.b32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}

// A thread-block cluster of S CTAs (S = 1, 2, 4 or 8) per token; CTA r of the cluster owns positions [r * span, (r + 1) * span) of the
// token's row.  out [T, k] int32: physical slot ids of the k best visible keys (keys above the k-th value in position order, then
// the ties that fill the list, also in position order), -1 padded.
//
// Three radix passes over the order-preserving key of the logit (11 + 11 + 10 bits).  Per pass every CTA histograms its span in
// shared memory, the cluster meets, every CTA adds up the S histograms through distributed shared memory and finds the digit
// of the k-th largest key with a block-wide prefix sum (thread i owns bins 2i and 2i + 1; exactly one bin b has
// count(bins > b) < remaining <= count(bins >= b)).  A serial walk down the 2048 bins by one thread took about as long as the
// histogram itself.  The list is then written by ordered compaction: spans in rank order (their counts are exchanged through
// distributed shared memory), 1024 positions at a time inside a span.
__global__ void __launch_bounds__(1024) indexer_topk_kernel(const float* __restrict__ logits, long long ld, const int* __restrict__ cu_seqlens_q,
                                                           const int* __restrict__ context_lens, int num_seqs, const int* __restrict__ block_tables,
                                                           int bt_stride, int bs, int k, int* __restrict__ out) {
  __shared__ int hist[2048];
  __shared__ int s_warp[32];
  __shared__ int s_cnt[2];                                   // keys of this span above / equal to the threshold
  __shared__ uint32_t s_prefix; __shared__ int s_remaining;
  const int S = (int)cluster_nctarank(), rank = (int)cluster_ctarank();
  const int t = blockIdx.x / S;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int lo = 0, hi = num_seqs;
  while (lo + 1 < hi) { int mid = (lo + hi) >> 1; if (cu_seqlens_q[mid] <= t) lo = mid; else hi = mid; }
  const int seq = lo;
  const int q_len = cu_seqlens_q[seq + 1] - cu_seqlens_q[seq];
  const int n = context_lens[seq] - q_len + (t - cu_seqlens_q[seq]) + 1;          // visible keys
  const float* row = logits + (long long)t * ld;
  const int* bt = block_tables ? block_tables + (long long)seq * bt_stride : nullptr;
  int* o = out + (long long)t * k;
  auto phys = [&](int idx) { return bt ? bt[idx / bs] * bs + idx % bs : idx; };
  if (n <= k) {                                               // uniform over the cluster: nobody waits at a cluster barrier below
    for (int i = rank * 1024 + tid; i < k; i += S * 1024) o[i] = i < n ? phys(i) : -1;
    return;
  }
  const int span = ((n + S - 1) / S + 3) & ~3;
  const int begin = min(n, rank * span), end = min(n, begin + span);
  const uint32_t hist_addr = smem_u32(hist);
  if (tid == 0) { s_prefix = 0; s_remaining = k; }
  const int shifts[3] = {21, 10, 0}, widths[3] = {11, 11, 10};
  uint32_t known_mask = 0;
  for (int p = 0; p < 3; p++) {
    for (int i = tid; i < 2048; i += 1024) hist[i] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    const int rem = s_remaining;
    const int sh = shifts[p];
    const uint32_t dm = (1u << widths[p]) - 1;
    for (int i = begin + tid; i < end; i += 1024) {
      const uint32_t key = float_key(row[i]);
      if ((key & known_mask) == prefix) atomicAdd(&hist[(key >> sh) & dm], 1);
    }
    __syncthreads();
    cluster_sync_all();                                       // every span's histogram is complete
    int c0 = 0, c1 = 0;
    for (int r = 0; r < S; r++) {
      const uint32_t a = mapa_shared(hist_addr + 8u * tid, (uint32_t)r);
      c0 += ld_dsmem_i32(a); c1 += ld_dsmem_i32(a + 4);
    }
    // inclusive prefix sum of the pair sums over the 1024 threads
    int incl = c0 + c1;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) { const int v = __shfl_up_sync(0xffffffffu, incl, d); if (lane >= d) incl += v; }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int w = s_warp[lane];
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) { const int v = __shfl_up_sync(0xffffffffu, w, d); if (lane >= d) w += v; }
      s_warp[lane] = w;
    }
    __syncthreads();
    const int total = s_warp[31];
    incl += warp > 0 ? s_warp[warp - 1] : 0;
    const int gt1 = total - incl, gt0 = gt1 + c1;             // keys in bins above 2i + 1 / above 2i
    if (gt1 < rem && rem <= gt1 + c1) { s_prefix = prefix | ((uint32_t)(2 * tid + 1) << sh); s_remaining = rem - gt1; }
    else if (gt0 < rem && rem <= gt0 + c0) { s_prefix = prefix | ((uint32_t)(2 * tid) << sh); s_remaining = rem - gt0; }
    known_mask |= dm << sh;
    __syncthreads();
    cluster_sync_all();                                       // everybody has read the histograms: they may be cleared
  }
  const uint32_t thr = s_prefix;                              // the k-th largest key; s_remaining of its copies are taken
  const int need_eq = s_remaining;
  const int n_gt = k - need_eq;
  // keys above / equal to the threshold in this span, then the offsets of the span in the two output groups
  int my_gt = 0, my_eq = 0;
  for (int i = begin + tid; i < end; i += 1024) {
    const uint32_t key = float_key(row[i]);
    my_gt += key > thr; my_eq += key == thr;
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) { my_gt += __shfl_xor_sync(0xffffffffu, my_gt, d); my_eq += __shfl_xor_sync(0xffffffffu, my_eq, d); }
  if (tid < 2) s_cnt[tid] = 0;
  __syncthreads();
  if (lane == 0) { atomicAdd(&s_cnt[0], my_gt); atomicAdd(&s_cnt[1], my_eq); }
  __syncthreads();
  cluster_sync_all();
  int base_gt = 0, base_eq = 0;
  const uint32_t cnt_addr = smem_u32(s_cnt);
  for (int r = 0; r < rank; r++) {
    const uint32_t a = mapa_shared(cnt_addr, (uint32_t)r);
    base_gt += ld_dsmem_i32(a); base_eq += ld_dsmem_i32(a + 4);
  }
  int* s_wgt = hist;
  int* s_weq = hist + 32;
  const unsigned lt = (1u << lane) - 1u;
  for (int i0 = begin; i0 < end && (base_gt < n_gt || base_eq < need_eq); i0 += 1024) {
    const int i = i0 + tid;
    const uint32_t key = i < end ? float_key(row[i]) : 0u;
    const bool gt = i < end && key > thr, eq = i < end && key == thr;
    const unsigned bg = __ballot_sync(0xffffffffu, gt), be = __ballot_sync(0xffffffffu, eq);
    if (lane == 0) { s_wgt[warp] = __popc(bg); s_weq[warp] = __popc(be); }
    __syncthreads();
    const int wg = s_wgt[lane], we = s_weq[lane];
    int ig = wg, ie = we;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int vg = __shfl_up_sync(0xffffffffu, ig, d), ve = __shfl_up_sync(0xffffffffu, ie, d);
      if (lane >= d) { ig += vg; ie += ve; }
    }
    const int tot_g = __shfl_sync(0xffffffffu, ig, 31), tot_e = __shfl_sync(0xffffffffu, ie, 31);
    const int off_g = __shfl_sync(0xffffffffu, ig - wg, warp), off_e = __shfl_sync(0xffffffffu, ie - we, warp);
    if (gt) {
      const int pos = base_gt + off_g + __popc(bg & lt);
      if (pos < n_gt) o[pos] = phys(i);
    } else if (eq) {
      const int pos = base_eq + off_e + __popc(be & lt);
      if (pos < need_eq) o[n_gt + pos] = phys(i);
    }
    base_gt += tot_g; base_eq += tot_e;
    __syncthreads();
  }
  cluster_sync_all();                                         // no CTA leaves while a peer may still read its counters
}

}  // namespace ne

using namespace ne;

// x [rows, 128] bf16 (row stride x_ld elements), heads = rows per token.  Keys: cache + slots given (q_out / s_out unused).
// Queries: q_out [rows, 128] e4m3 + s_out [rows].
extern "C" int ne_indexer_prep(const void* x, long long x_ld, int rows, int heads, const void* ln_w, const void* ln_b, float eps,
                               const long long* positions, const float* rope_cache, int rope, void* q_out, float* s_out, void* cache,
                               const long long* slots, int bs, long long page_bytes, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (heads < 1 || rows % heads || rope < 8 || rope > kIdxD || (rope & (rope - 1)) || x_ld % 4) return 1001;
  if (!cache && (!q_out || !s_out)) return 1002;
  indexer_prep_kernel<<<(rows + 7) / 8, 256, 0, st>>>((const __nv_bfloat16*)x, x_ld, rows, heads, (const __nv_bfloat16*)ln_w, (const __nv_bfloat16*)ln_b, eps,
                                                      positions, rope_cache, rope, (uint8_t*)q_out, s_out, (uint8_t*)cache, slots, bs, page_bytes);
  return (int)cudaGetLastError();
}

// q8 [T * heads, 128] e4m3; cache [num_blocks, page_bytes] with page = [64 x 128 B keys | 64 fp32 scales]; logits [T, ld] fp32
// (ld a multiple of 4, at least the largest context rounded up to 128).  Columns past a token's causal limit inside its last
// tile are written as -inf; columns in later tiles are left untouched.
extern "C" int ne_indexer_logits(const void* q8, const float* q_scale, const float* head_w, const void* cache, int num_blocks, long long page_bytes,
                                 const int* block_tables, int bt_stride, const int* cu_seqlens_q, const int* context_lens, int num_seqs,
                                 int T, int heads, int splits, float* logits, long long ld, cudaStream_t st) {
  if (T <= 0) return 0;
  if (heads < 1 || heads > 64 || splits < 1 || page_bytes != kIdxPage * (kIdxD + 4) || ld % 4) return 1001;
  CUtensorMap tq, tk;
  {
    uint64_t dims[2] = {kIdxD, (uint64_t)T * heads}; uint64_t strides[1] = {kIdxD}; uint32_t box[2] = {kIdxD, 64};
    int rc = make_tmap(&tq, q8, TMA_U8, 2, dims, strides, box, TMA_SW_128); if (rc) return 2000 + rc;
  }
  {
    uint64_t dims[3] = {kIdxD, kIdxPage, (uint64_t)num_blocks}; uint64_t strides[2] = {kIdxD, (uint64_t)page_bytes}; uint32_t box[3] = {kIdxD, kIdxPage, 1};
    int rc = make_tmap(&tk, cache, TMA_U8, 3, dims, strides, box, TMA_SW_128); if (rc) return 2100 + rc;
  }
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(indexer_logits_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kIdxSmem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  IdxArgs a;
  a.head_w = head_w; a.q_scale = q_scale; a.cache = (const uint8_t*)cache; a.page_bytes = page_bytes; a.block_tables = block_tables;
  a.bt_stride = bt_stride; a.cu_seqlens_q = cu_seqlens_q; a.context_lens = context_lens; a.num_seqs = num_seqs; a.T = T; a.heads = heads;
  a.splits = splits; a.logits = logits; a.ld = ld;
  indexer_logits_kernel<<<dim3((unsigned)T, (unsigned)splits), kIdxThreads, kIdxSmem, st>>>(tq, tk, a);
  return (int)cudaGetLastError();
}

extern "C" int ne_indexer_topk(const float* logits, long long ld, const int* cu_seqlens_q, const int* context_lens, int num_seqs,
                               const int* block_tables, int bt_stride, int bs, int k, int T, int* out, cudaStream_t st) {
  if (T <= 0) return 0;
  if (k < 1 || bs < 1) return 1001;
  // few tokens over long rows: several CTAs share a row (a cluster per token), as many as keeps every CTA at >= 8192 positions and
  // the grid within one wave
  int S = 1;
  while (S < 8 && T * S * 2 <= 148 && ld / (S * 2) >= 8192) S *= 2;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(T * S), 1, 1);
  cfg.blockDim = dim3(1024, 1, 1);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)S; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, indexer_topk_kernel, logits, ld, cu_seqlens_q, context_lens, num_seqs, block_tables, bt_stride, bs, k, out);
}
