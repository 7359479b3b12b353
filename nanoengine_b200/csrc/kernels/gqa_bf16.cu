// Grouped-query paged attention on tcgen05 tensor cores: bf16 queries, bf16 paged K / V caches, head dim 128, 64-token
// pages.  Serves decode (q_len 1..N+1) and prefill / chunked prefill alike.
//
// One CTA = one KV head x one tile of 128 query rows of ONE sequence x one slice of its key pages.  A row is a
// (token, query head of the group) pair, r = token_in_tile * g + head_in_group with g = Hq / Hkv (a power of two up to
// 128), so a decode token of Qwen3 (g = 16) fills 16 rows and a prefill tile carries 128 / g consecutive tokens that all
// reuse the same K / V pages.  Every row has its own causal limit.
//
// Per 64-key page:  S = Q K^T   (8 x tcgen05.mma kind::f16, M=128 N=64 K=16, both operands K-major, 128B swizzle)
//                   online softmax by 128 threads (one per row) reading S from TMEM; P -> bf16 -> smem
//                   O += P V    (4 x tcgen05.mma, M=128 N=128 K=16; V is read MN-major from its page tile)
// TMEM: S double-buffered (2 x 64 columns) + O (128 columns).  Shared memory: Q 32 KB, 3 stages of K+V 32 KB, P 2 x 16 KB.
// Warp 0: TMA producer, warp 1: MMA issuer, warps 2-5: softmax / rescale / epilogue.  All waits are bounded.
// With more than one key slice the CTA writes a normalised partial result and its log2-sum-exp; ne_attn_merge folds them.
//
// Replaces in the reference: flashinfer trtllm_batch_decode_with_kv_cache and flash_attn.cute varlen prefill
// (layers/backends/attention/fa4.py:34-245), FA3 / FA2 / FlashInfer wrappers (attention/fa3.py, fa2.py, base.py:132-280).
#include "ptx.cuh"
#include "tma_host.h"

namespace ne {

constexpr int kGqaThreads = 192;
constexpr int kKernelGqa = 7;
constexpr int kGD = 128;                     // head dim
constexpr int kGPage = 64;                   // keys per page
constexpr int kGVBytes = kGPage * kGD * 2;   // 16 KB per V tile (and per K tile of a 128-wide head)
constexpr int kGStages = 3;
constexpr int kGPBytes = 128 * 128;          // P tile: 128 rows x 64 bf16
// kC = 64-element chunks of the query / key head dim: 2 (grouped-query models, head dim 128) or 3 (the non-absorbed form of MLA:
// 128 no-position dims + 64 rotary dims = 192; values stay 128 wide)
template <int kC> struct GqaSmem {
  static constexpr int kQ = 128 * 64 * 2 * kC;        // Q tile: kC chunks of 128 rows x 128 B
  static constexpr int kK = kGPage * 64 * 2 * kC;     // K tile: kC chunks of 64 keys x 128 B
  static constexpr int kStage = kK + kGVBytes;
  static constexpr int kBytes = kQ + kGStages * kStage + 2 * kGPBytes + 1024 + 256;
};

struct GqaArgs {
  const int* block_tables; int bt_stride;
  const int* cu_seqlens_q; const int* context_lens; int num_seqs;
  int T, Hq, Hkv, g, tq, splits;             // g = Hq / Hkv, tq = 128 / g query tokens per tile
  float scale_log2;
  __nv_bfloat16* out;                        // [T, Hq, 128] (splits == 1)
  float* part; float* lse2;                  // [splits, T, Hq, 128], [splits, T, Hq] (splits > 1)
};

// kRagged: keys and values are not paged.  They are the rows of the same tokens as the queries (a prompt without a cached
// prefix): K no-position part [T, H, 128] and V [T, H, 128] contiguous, the rotary part of the key [T, 64] shared by all heads.
// "Page" i of a sequence is then its tokens [64 i, 64 i + 64), fetched by token coordinate; rows past the sequence's end belong
// to the next sequence and are masked by the causal limit like any later key.

template <int kC, bool kRagged>
__global__ void __launch_bounds__(kGqaThreads, 1)
gqa_bf16_kernel(const __grid_constant__ CUtensorMap tq_map, const __grid_constant__ CUtensorMap tk_map, const __grid_constant__ CUtensorMap tv_map,
                const __grid_constant__ CUtensorMap tr_map, const GqaArgs a) {
  constexpr int kGQBytes = GqaSmem<kC>::kQ, kGKBytes = GqaSmem<kC>::kK, kStage = GqaSmem<kC>::kStage;
  pdl_wait(); pdl_trigger();      // dependent launch: nothing above this line touches global memory
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sKV = sQ + kGQBytes;                                     // per stage: [K kC x 8 KB][V 16 KB]
  uint8_t* sP = sKV + kGStages * kStage;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * kGPBytes);
  // q_full | kv_full[3] | kv_empty[3] | s_full[2] | s_empty[2] | p_full[2] | p_empty[2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_tile = reinterpret_cast<int*>(tmem_slot + 2);              // [seq, first token of the tile (global index)]
  const uint32_t b_qfull = smem_u32(bars), b_kvfull = smem_u32(bars + 1), b_kvempty = smem_u32(bars + 4);
  const uint32_t b_sfull = smem_u32(bars + 7), b_sempty = smem_u32(bars + 9), b_pfull = smem_u32(bars + 11), b_pempty = smem_u32(bars + 13);

  const int warp = threadIdx.x >> 5;
  const int hkv = blockIdx.y, split = blockIdx.z;

  // which sequence and which of its token tiles is this CTA?  Tiles never straddle sequences.
  // (warp 0 searches 32 sequences per round with a prefix sum of their tile counts: one thread walking the sequences
  // delays the CTAs of the last sequences of a 256-sequence decode batch by several microseconds)
  if (warp == 0) {
    const int lane = (int)lane_id();
    int rem = blockIdx.x, seq = -1, tok0 = 0;
    for (int s0 = 0; s0 < a.num_seqs && seq < 0; s0 += 32) {
      const int s = s0 + lane;
      int q0 = 0, nt = 0;
      if (s < a.num_seqs) { q0 = a.cu_seqlens_q[s]; nt = (a.cu_seqlens_q[s + 1] - q0 + a.tq - 1) / a.tq; }
      int incl = nt;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) { const int v = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += v; }
      const unsigned hit = __ballot_sync(0xffffffffu, rem < incl);        // lanes whose running count passes the tile index
      if (hit) {
        const int l = __ffs(hit) - 1;
        const int before = __shfl_sync(0xffffffffu, incl - nt, l);
        seq = s0 + l;
        tok0 = __shfl_sync(0xffffffffu, q0, l) + (rem - before) * a.tq;
      } else {
        rem -= __shfl_sync(0xffffffffu, incl, 31);
      }
    }
    if (lane == 0) { s_tile[0] = seq; s_tile[1] = tok0; }
  }
  if (threadIdx.x == 0) {
    mbar_init(b_qfull, 1);
    for (int i = 0; i < kGStages; i++) { mbar_init(b_kvfull + 8 * i, 1); mbar_init(b_kvempty + 8 * i, 1); }
    for (int i = 0; i < 2; i++) { mbar_init(b_sfull + 8 * i, 1); mbar_init(b_sempty + 8 * i, 4); }
    for (int i = 0; i < 2; i++) { mbar_init(b_pfull + 8 * i, 4); mbar_init(b_pempty + 8 * i, 1); }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 128;
  const int seq = s_tile[0], tok0 = s_tile[1];

  // geometry of the tile (uniform over the CTA); a CTA past the last tile has nothing to do
  int n_tiles = 0, pg_begin = 0, n_tok = 0, base_limit = -1;
  const int* bt = a.block_tables;
  if (seq >= 0) {
    const int q_beg = a.cu_seqlens_q[seq], q_len = a.cu_seqlens_q[seq + 1] - q_beg;
    n_tok = min(a.tq, q_beg + q_len - tok0);
    base_limit = a.context_lens[seq] - q_len + (tok0 - q_beg);              // last key visible to the tile's first token
    const int max_limit = base_limit + n_tok - 1;                            // ... to its last token
    const int total_pages = max_limit >= 0 ? max_limit / kGPage + 1 : 0;
    const int per_split = (total_pages + a.splits - 1) / a.splits;
    pg_begin = split * per_split;
    n_tiles = max(0, min(total_pages, pg_begin + per_split) - pg_begin);
    bt = a.block_tables + (long long)seq * a.bt_stride;
  }

  if (warp == 0) {
    if (n_tiles > 0 && elect_one()) {
      mbar_expect_tx(b_qfull, kGQBytes);
      // box {64 elems, g heads, tq tokens, kC chunks}: lands as [chunk][token][head][128 B], i.e. row = token * g + head
      tma_load_4d(smem_u32(sQ), &tq_map, b_qfull, 0, hkv * a.g, tok0, 0);
      const int k_beg = kRagged ? a.cu_seqlens_q[seq] : 0;
      for (int i = 0; i < n_tiles; i++) {
        const int s = i % kGStages;
        if (!mbar_wait(b_kvempty + 8 * s, ((i / kGStages) & 1) ^ 1, abort_flag, kKernelGqa, 100 + s)) break;
        uint8_t* dst = sKV + s * kStage;
        mbar_expect_tx(b_kvfull + 8 * s, kStage);
        if (kRagged) {
          const int tok = k_beg + (pg_begin + i) * kGPage;                 // rows past the tensor's end are zero-filled
          tma_load_4d(smem_u32(dst), &tk_map, b_kvfull + 8 * s, 0, tok, hkv, 0);                    // no-position part: 2 chunks
          tma_load_2d(smem_u32(dst + 2 * kGPage * 128), &tr_map, b_kvfull + 8 * s, 0, tok);         // rotary part: third chunk
          tma_load_4d(smem_u32(dst + kGKBytes), &tv_map, b_kvfull + 8 * s, 0, tok, hkv, 0);
        } else {
          int block = bt[pg_begin + i];
          if (!NE_INDEX_OK(block, BK_CACHE_PAGES, 7, __LINE__)) block = 0;      // a bad page id reads page 0 instead of another allocation
          tma_load_5d(smem_u32(dst), &tk_map, b_kvfull + 8 * s, 0, 0, hkv, block, 0);
          tma_load_5d(smem_u32(dst + kGKBytes), &tv_map, b_kvfull + 8 * s, 0, 0, hkv, block, 0);
        }
      }
    }
  } else if (warp == 1) {
    if (n_tiles > 0 && elect_one()) {
      constexpr uint32_t kIdescQK = make_idesc(FMT_BF16, FMT_BF16, 128, kGPage);
      constexpr uint32_t kIdescPV = make_idesc(FMT_BF16, FMT_BF16, 128, kGD, 0, 1);      // B (= V) is MN-major
      bool ok = mbar_wait(b_qfull, 0, abort_flag, kKernelGqa, 200);
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      auto pv = [&](int j) -> bool {
        if (!mbar_wait(b_pfull + 8 * (j & 1), (j >> 1) & 1, abort_flag, kKernelGqa, 230)) return false;
        tc_fence_after();
        const int s = j % kGStages;
        const uint32_t vt = smem_u32(sKV + s * kStage + kGKBytes);
#pragma unroll
        for (int ks = 0; ks < 4; ks++) {                     // 16 keys per MMA
          uint64_t adesc = make_smem_desc(p_addr + (j & 1) * kGPBytes + ks * 32, 16, 1024, SW_128B);
          uint64_t bdesc = make_smem_desc(vt + ks * 16 * 128, kGPage * 128, 1024, SW_128B);
          umma_f16(tmem_o, adesc, bdesc, kIdescPV, (j | ks) != 0);
        }
        tc_commit(b_kvempty + 8 * s);
        tc_commit(b_pempty + 8 * (j & 1));
        return true;
      };
      // the barriers that gate S(i+1) are tested before the MMAs of S(i) are issued: a test costs ~150 cycles even when the
      // phase completed long ago, and issuing MMAs blocks for about as long as they run, which hides it
      bool pre_se = true, pre_kv = mbar_test(b_kvfull, 0);
      for (int i = 0; ok && i < n_tiles; i++) {
        const int sb = i & 1, s = i % kGStages;
        if (!pre_se && !mbar_wait(b_sempty + 8 * sb, ((i >> 1) & 1) ^ 1, abort_flag, kKernelGqa, 210 + sb)) { ok = false; break; }
        if (!pre_kv && !mbar_wait(b_kvfull + 8 * s, (i / kGStages) & 1, abort_flag, kKernelGqa, 220 + s)) { ok = false; break; }
        mbar_test2(b_sempty + 8 * ((i + 1) & 1), (((i + 1) >> 1) & 1) ^ 1, b_kvfull + 8 * ((i + 1) % kGStages), ((i + 1) / kGStages) & 1,
                   pre_se, pre_kv);
        tc_fence_after();
        const uint32_t kt = smem_u32(sKV + s * kStage);
        const uint32_t d = tmem_base + sb * kGPage;
#pragma unroll
        for (int c = 0; c < kC; c++) {                       // 64-element chunks of the query / key head dim
#pragma unroll
          for (int ks = 0; ks < 4; ks++) {
            uint64_t adesc = make_smem_desc(q_addr + c * 128 * 128 + ks * 32, 16, 1024, SW_128B);
            uint64_t bdesc = make_smem_desc(kt + c * kGPage * 128 + ks * 32, 16, 1024, SW_128B);
            umma_f16(d, adesc, bdesc, kIdescQK, (c | ks) != 0);
          }
        }
        tc_commit(b_sfull + 8 * sb);
        if (i > 0 && !pv(i - 1)) { ok = false; break; }
      }
      if (ok) pv(n_tiles - 1);
    }
  } else {
    const int wq = warp & 3;
    const int row = wq * 32 + (int)lane_id();
    const uint32_t lane_addr = (uint32_t)(wq * 32) << 16;
    const int tl = row / a.g, hg = row % a.g;                 // token in tile, head in group
    const bool row_ok = tl < n_tok;
    const int limit = row_ok ? base_limit + tl : -1;          // this row's last visible key
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    bool s_ready = false;                            // early test of the next page's S buffer
    for (int i = 0; ok && i < n_tiles; i++) {
      const int sb = i & 1;
      if (!s_ready && !mbar_wait(b_sfull + 8 * sb, (i >> 1) & 1, abort_flag, kKernelGqa, 300 + sb)) { ok = false; break; }
      tc_fence_after();
      uint32_t r0[32], r1[32];
      tmem_ld_32x32b_x32(tmem_base + lane_addr + sb * kGPage, r0);
      tmem_ld_32x32b_x32(tmem_base + lane_addr + sb * kGPage + 32, r1);
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane_id() == 0) mbar_arrive(b_sempty + 8 * sb);
      const int key0 = (pg_begin + i) * kGPage;
      const bool p_free = i < 2 || mbar_test(b_pempty + 8 * (i & 1), ((i - 2) >> 1) & 1);     // needed only after the math
      if (key0 + kGPage - 1 > limit) {
#pragma unroll
        for (int j = 0; j < 32; j++) {
          if (key0 + j > limit) r0[j] = 0xff800000u;
          if (key0 + 32 + j > limit) r1[j] = 0xff800000u;
        }
      }
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        mx[0] = fmaxf(mx[0], __uint_as_float(r0[j])); mx[1] = fmaxf(mx[1], __uint_as_float(r0[j + 1]));
        mx[2] = fmaxf(mx[2], __uint_as_float(r1[j])); mx[3] = fmaxf(mx[3], __uint_as_float(r1[j + 1]));
      }
      const float m_tile = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * a.scale_log2;
      // lazy rescaling: the reference maximum only moves when the page's maximum exceeds it by more than 2^8
      const bool first_valid = (m_run == -INFINITY);
      const float m_new = (first_valid || m_tile > m_run + 8.f) ? fmaxf(m_run, m_tile) : m_run;
      const float alpha = (m_new == -INFINITY || first_valid) ? 1.f : exp2f(m_run - m_new);
      const float neg_m = (m_new == -INFINITY) ? 0.f : -m_new;
      float psum = 0.f;
      uint32_t pk[32];
#pragma unroll
      for (int j = 0; j < 16; j++) {
        const float p0 = exp2f(fmaf(__uint_as_float(r0[2 * j]), a.scale_log2, neg_m)), p1 = exp2f(fmaf(__uint_as_float(r0[2 * j + 1]), a.scale_log2, neg_m));
        const float p2 = exp2f(fmaf(__uint_as_float(r1[2 * j]), a.scale_log2, neg_m)), p3 = exp2f(fmaf(__uint_as_float(r1[2 * j + 1]), a.scale_log2, neg_m));
        pk[j] = pack_bf16x2(p0, p1);
        pk[16 + j] = pack_bf16x2(p2, p3);
        // sum what the MMA will see (bf16-rounded probabilities), so numerator and denominator stay consistent
        const float2 q0 = unpack_bf16x2(pk[j]), q1 = unpack_bf16x2(pk[16 + j]);
        psum += (q0.x + q0.y) + (q1.x + q1.y);
      }
      l_run = l_run * alpha + psum;
      m_run = m_new;
      if (i > 0 && __any_sync(0xffffffffu, alpha < 1.f)) {
        if (!mbar_wait(b_pempty + 8 * ((i - 1) & 1), ((i - 1) >> 1) & 1, abort_flag, kKernelGqa, 310)) { ok = false; break; }
        tc_fence_after();
#pragma unroll 1
        for (int cblk = 0; cblk < kGD / 16; cblk++) {
          uint32_t o[16];
          tmem_ld_32x32b_x16(tmem_o + lane_addr + cblk * 16, o);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; j++) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
          tmem_st_32x32b_x16(tmem_o + lane_addr + cblk * 16, o);
        }
        tc_wait_st();
      }
      if (!p_free && !mbar_wait(b_pempty + 8 * (i & 1), ((i - 2) >> 1) & 1, abort_flag, kKernelGqa, 311)) { ok = false; break; }
      s_ready = mbar_test(b_sfull + 8 * ((i + 1) & 1), ((i + 1) >> 1) & 1);
      // P row (64 bf16 = 8 chunks of 16 bytes) into the 128B-swizzled K-major layout the MMA reads
      {
        uint8_t* prow = sP + (i & 1) * kGPBytes + row * 128;
        const int sw = row & 7;
#pragma unroll
        for (int cch = 0; cch < 8; cch++)
          *reinterpret_cast<uint4*>(prow + ((cch ^ sw) << 4)) = make_uint4(pk[4 * cch], pk[4 * cch + 1], pk[4 * cch + 2], pk[4 * cch + 3]);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane_id() == 0) mbar_arrive(b_pfull + 8 * (i & 1));
    }
    if (ok && n_tiles > 0) ok = mbar_wait(b_pempty + 8 * ((n_tiles - 1) & 1), ((n_tiles - 1) >> 1) & 1, abort_flag, kKernelGqa, 320);
    const long long orow = row_ok ? ((long long)(tok0 + tl) * a.Hq + hkv * a.g + hg) : 0;
    if (ok && n_tiles > 0) {
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
#pragma unroll 1
      for (int cblk = 0; cblk < kGD / 32; cblk++) {
        uint32_t o[32];
        tmem_ld_32x32b_x32(tmem_o + lane_addr + cblk * 32, o);
        tc_wait_ld();
        if (row_ok) {
          if (a.splits == 1) {
            __nv_bfloat16* dst = a.out + orow * kGD + cblk * 32;
#pragma unroll
            for (int v = 0; v < 4; v++) {
              *reinterpret_cast<uint4*>(dst + v * 8) = make_uint4(
                  pack_bf16x2(__uint_as_float(o[v * 8]) * inv, __uint_as_float(o[v * 8 + 1]) * inv),
                  pack_bf16x2(__uint_as_float(o[v * 8 + 2]) * inv, __uint_as_float(o[v * 8 + 3]) * inv),
                  pack_bf16x2(__uint_as_float(o[v * 8 + 4]) * inv, __uint_as_float(o[v * 8 + 5]) * inv),
                  pack_bf16x2(__uint_as_float(o[v * 8 + 6]) * inv, __uint_as_float(o[v * 8 + 7]) * inv));
            }
          } else {
            float* dst = a.part + ((long long)split * a.T * a.Hq + orow) * kGD + cblk * 32;
#pragma unroll
            for (int v = 0; v < 8; v++)
              *reinterpret_cast<float4*>(dst + v * 4) = make_float4(__uint_as_float(o[v * 4]) * inv, __uint_as_float(o[v * 4 + 1]) * inv,
                                                                    __uint_as_float(o[v * 4 + 2]) * inv, __uint_as_float(o[v * 4 + 3]) * inv);
          }
        }
      }
    }
    if (a.splits > 1 && row_ok)
      a.lse2[(long long)split * a.T * a.Hq + orow] = (ok && n_tiles > 0 && l_run > 0.f) ? m_run + log2f(l_run) : -INFINITY;
    if (a.splits > 1 && row_ok && n_tiles == 0) {
      float* dst = a.part + ((long long)split * a.T * a.Hq + orow) * kGD;
      for (int c = 0; c < kGD; c += 4) *reinterpret_cast<float4*>(dst + c) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (a.splits == 1 && n_tiles == 0 && row_ok) {
      __nv_bfloat16* dst = a.out + orow * kGD;
      for (int c = 0; c < kGD; c += 8) *reinterpret_cast<uint4*>(dst + c) = make_uint4(0, 0, 0, 0);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) for (int i = 0; i < 2000; i++) __nanosleep(1000);
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 256); }
}

}  // namespace ne

using namespace ne;

// q bf16 [T, Hq, 128] (contiguous), k_cache / v_cache bf16 [num_blocks, 64, Hkv, 128].  max_tiles = an upper bound of
// sum over sequences of ceil(q_len / (128 / g)) known on the host (e.g. T for decode, ceil(T / tq) + num_seqs in general).
extern "C" int ne_gqa_bf16(const void* q, const void* k_cache, const void* v_cache, int num_blocks, const int* block_tables, int bt_stride,
                           const int* cu_seqlens_q, const int* context_lens, int num_seqs, int T, int Hq, int Hkv, int max_tiles, int splits,
                           float scale, void* out, float* part, float* lse2, cudaStream_t st) {
  if (T <= 0) return 0;
  if (Hkv < 1 || Hq % Hkv || splits < 1 || (splits > 1 && (!part || !lse2))) return 1001;
  const int g = Hq / Hkv;
  if (g > 128 || (g & (g - 1))) return 1002;
  const int tq = 128 / g;
  CUtensorMap mq, mk, mv;
  {
    // {64 elems, heads, tokens, 2 chunks}; the chunk stride (128 B) is smaller than the head stride, which the encoder accepts
    uint64_t dims[4] = {64, (uint64_t)Hq, (uint64_t)T, 2}; uint64_t strides[3] = {(uint64_t)kGD * 2, (uint64_t)Hq * kGD * 2, 128};
    uint32_t box[4] = {64, (uint32_t)g, (uint32_t)tq, 2};
    int rc = make_tmap(&mq, q, TMA_BF16, 4, dims, strides, box, TMA_SW_128); if (rc) return 2000 + rc;
  }
  for (int which = 0; which < 2; which++) {
    uint64_t dims[5] = {64, (uint64_t)kGPage, (uint64_t)Hkv, (uint64_t)num_blocks, 2};
    uint64_t strides[4] = {(uint64_t)Hkv * kGD * 2, (uint64_t)kGD * 2, (uint64_t)kGPage * Hkv * kGD * 2, 128};
    uint32_t box[5] = {64, kGPage, 1, 1, 2};
    int rc = make_tmap(which ? &mv : &mk, which ? v_cache : k_cache, TMA_BF16, 5, dims, strides, box, TMA_SW_128); if (rc) return 2100 + rc;
  }
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gqa_bf16_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, GqaSmem<2>::kBytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  GqaArgs a;
  a.block_tables = block_tables; a.bt_stride = bt_stride; a.cu_seqlens_q = cu_seqlens_q; a.context_lens = context_lens; a.num_seqs = num_seqs;
  a.T = T; a.Hq = Hq; a.Hkv = Hkv; a.g = g; a.tq = tq; a.splits = splits; a.scale_log2 = scale * 1.4426950408889634f;
  a.out = (__nv_bfloat16*)out; a.part = part; a.lse2 = lse2;
  return (int)launch_pdl(gqa_bf16_kernel<2, false>, dim3(dim3((unsigned)max_tiles, (unsigned)Hkv, (unsigned)splits)), dim3(kGqaThreads), GqaSmem<2>::kBytes,
                         st, mq, mk, mv, mk, a);
}

// Non-absorbed MLA attention of prompts without a cached prefix (causal, ragged): q bf16 [T, H, 192] (row stride q_ld elements; the last
// 64 dims rotated), k_nope bf16 [T, H, 128] and v bf16 [T, H, 128] contiguous, k_rope bf16 [T, 64] (row stride kr_ld elements) shared by
// the heads, cu_seqlens [num_seqs + 1] (queries and keys alike).  out bf16 [T, H, 128].  max_tiles >= sum of ceil(len / 128).
// Replaces in the reference: the FA4 ragged prefill call of models/deepseek_v2/deepseek_v2.py:1792-1816.
extern "C" int ne_mla_prefill_bf16(const void* q, long long q_ld, const void* k_nope, const void* k_rope, long long kr_ld, const void* v,
                                   const int* cu_seqlens, const int* seq_lens, int num_seqs, int T, int H, int max_tiles, float scale, void* out,
                                   cudaStream_t st) {
  if (T <= 0) return 0;
  if (H < 1 || q_ld % 8 || kr_ld % 8 || q_ld < (long long)H * 192) return 1001;
  CUtensorMap mq, mk, mv, mr;
  {
    uint64_t dims[4] = {64, (uint64_t)H, (uint64_t)T, 3}; uint64_t strides[3] = {192 * 2, (uint64_t)q_ld * 2, 128};
    uint32_t box[4] = {64, 1, 128, 3};
    int rc = make_tmap(&mq, q, TMA_BF16, 4, dims, strides, box, TMA_SW_128); if (rc) return 2000 + rc;
  }
  for (int which = 0; which < 2; which++) {
    // {64 elems, tokens, heads, 2 chunks}: a box of 64 tokens of one head lands as [chunk][token][128 B]
    uint64_t dims[4] = {64, (uint64_t)T, (uint64_t)H, 2}; uint64_t strides[3] = {(uint64_t)H * 128 * 2, 128 * 2, 128};
    uint32_t box[4] = {64, kGPage, 1, 2};
    int rc = make_tmap(which ? &mv : &mk, which ? v : k_nope, TMA_BF16, 4, dims, strides, box, TMA_SW_128); if (rc) return 2100 + rc;
  }
  {
    uint64_t dims[2] = {64, (uint64_t)T}; uint64_t strides[1] = {(uint64_t)kr_ld * 2}; uint32_t box[2] = {64, kGPage};
    int rc = make_tmap(&mr, k_rope, TMA_BF16, 2, dims, strides, box, TMA_SW_128); if (rc) return 2200 + rc;
  }
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gqa_bf16_kernel<3, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, GqaSmem<3>::kBytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  GqaArgs a;
  a.block_tables = nullptr; a.bt_stride = 0; a.cu_seqlens_q = cu_seqlens; a.context_lens = seq_lens; a.num_seqs = num_seqs;
  a.T = T; a.Hq = H; a.Hkv = H; a.g = 1; a.tq = 128; a.splits = 1; a.scale_log2 = scale * 1.4426950408889634f;
  a.out = (__nv_bfloat16*)out; a.part = nullptr; a.lse2 = nullptr;
  return (int)launch_pdl(gqa_bf16_kernel<3, true>, dim3(dim3((unsigned)max_tiles, (unsigned)H, 1)), dim3(kGqaThreads), GqaSmem<3>::kBytes, st, mq, mk, mv,
                         mr, a);
}
