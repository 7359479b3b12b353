// Absorbed MLA attention over the paged fp8 latent cache on tcgen05 tensor cores (DeepSeek-V3 geometry: 576-value
// rows = 512 latent + 64 rope, 512-value output, 64-token pages).  Serves decode (q_len 1..N+1) and absorbed prefill
// alike: one CTA handles the heads (<= 128) of ONE query token, one half (256 values) of the output width and one
// slice of the key pages; keys are causal-limited per token, so a prefix-cache hit or a chunked prefill needs no
// separate gather/merge pass.
//
// Per 64-token page:  S = Q K^T   (18 x tcgen05.mma kind::f8f6f4, M=128 N=64 K=32, both operands K-major in smem)
//                     online softmax by 128 threads (one per head) reading S from TMEM; P -> e4m3 -> smem
//                     O += P V    (2 x tcgen05.mma, V is the same page tile read MN-major, N=256)
// TMEM: S double-buffered (2 x 64 columns) + O (256 columns).  Shared memory: Q 72 KB, 3-page ring 108 KB, P 2 x 8 KB.
// Warp 0: TMA producer; warp 1: MMA issuer; warps 2-5: softmax / rescale / epilogue.  All waits are bounded.
// With more than one key slice the CTA writes a normalised partial result and its log2-sum-exp; ne_attn_merge folds them.
//
// Sparse form (DSA): the keys of a token are not pages but a list of cache rows picked by the lightning indexer (top-k
// physical slot ids, -1 = none).  The same pipeline runs over tiles of 64 listed rows; only the producer differs: warp 0
// gathers the 64 rows (576 bytes each, 16 bytes per cp.async) into the swizzled layout TMA would have produced, zero-filling
// rows without an id, and hands a tile over once its copies have landed and were fenced for the tensor-core proxy.  The
// softmax warps mask the columns whose id is -1.  This is the tensor-core replacement for the CUDA-core gather path
// (reference layers/backends/mla/trtllm.py:93-204 `sparse_mla_top_k`, layers/backends/mla/flash_mla.py:22-121).
//
// fp8 contract (reference layers/backends/mla/trtllm.py:93-204): the query is clamped to +-448 and cast to e4m3 without
// a scale, cache rows are clamped-cast e4m3, softmax scale is applied to the fp32 logits.
#include <atomic>

#include "ptx.cuh"
#include "tma_host.h"

namespace ne {

constexpr int kMlaThreads = 192;
constexpr int kMlaSparseThreads = 288;        // + three more gather warps
constexpr int kKernelMla = 2;
constexpr int kPage = 64, kDk = 576, kDv = 512, kVHalf = 256;
constexpr int kQNope = 4 * 128 * 128;          // four 128-byte-wide panels of 128 rows
constexpr int kQBytes = kQNope + 128 * 64;     // + rope panel (64 bytes wide)
constexpr int kPgNope = 4 * kPage * 128;
constexpr int kPgBytes = kPgNope + kPage * 64;
constexpr int kPgStages = 3;
constexpr int kPBytes = 128 * 64;      // one P buffer; two are kept so softmax of page i+1 overlaps P V of page i
constexpr int kMlaSmem = kQBytes + kPgStages * kPgBytes + 2 * kPBytes + 1024 + 256;

struct MlaArgs {
  const int* block_tables; int bt_stride;
  const int* cu_seqlens_q; const int* context_lens; int num_seqs;
  int T, H, splits;
  float scale_log2;                  // softmax scale * log2(e)
  __nv_bfloat16* out;                // [T, H, 512] (splits == 1)
  float* part; float* lse2;          // [splits, T, H, 512], [splits, T, H] (splits > 1)
  // sparse form
  const int* sparse; int topk;       // [T, topk] cache row ids (block * 64 + offset), -1 = no key
  const uint8_t* cache; long long cache_rows;
};

template <bool kSparse>
__global__ void __launch_bounds__(kSparse ? kMlaSparseThreads : kMlaThreads, 1)
mla_fp8_kernel(const __grid_constant__ CUtensorMap tq128, const __grid_constant__ CUtensorMap tq64,
               const __grid_constant__ CUtensorMap tk128, const __grid_constant__ CUtensorMap tk64, const MlaArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sPg = sQ + kQBytes;
  uint8_t* sP = sPg + kPgStages * kPgBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * kPBytes);
  // q_full | pg_full[3] | pg_empty[3] | s_full[2] | s_empty[2] | p_full[2] | p_empty[2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t b_qfull = smem_u32(bars), b_pgfull = smem_u32(bars + 1), b_pgempty = smem_u32(bars + 4);
  const uint32_t b_sfull = smem_u32(bars + 7), b_sempty = smem_u32(bars + 9), b_pfull = smem_u32(bars + 11), b_pempty = smem_u32(bars + 13);

  const int warp = threadIdx.x >> 5;
  // the two output halves of a token sit in adjacent CTAs so the second reader of every KV page hits L2
  const int t = blockIdx.x >> 1, vhalf = blockIdx.x & 1, split = blockIdx.y;

  if (threadIdx.x == 0) {
    mbar_init(b_qfull, 1);
    for (int i = 0; i < kPgStages; i++) { mbar_init(b_pgfull + 8 * i, kSparse ? 128 : 1); mbar_init(b_pgempty + 8 * i, 1); }
    for (int i = 0; i < 2; i++) { mbar_init(b_sfull + 8 * i, 1); mbar_init(b_sempty + 8 * i, 4); }
    for (int i = 0; i < 2; i++) { mbar_init(b_pfull + 8 * i, 4); mbar_init(b_pempty + 8 * i, 1); }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), 512); tmem_relinquish(); }
  pdl_wait(); pdl_trigger();      // dependent launch: the set-up above touches no global memory

  // sequence of this token, causal limit, page range of this split (uniform over the CTA)
  int seq = 0, limit = 0x3fffffff, total_pages;
  const int* bt = nullptr;
  if (!kSparse) {
    int lo = 0, hi = a.num_seqs;
    while (lo + 1 < hi) { int mid = (lo + hi) >> 1; if (a.cu_seqlens_q[mid] <= t) lo = mid; else hi = mid; }
    seq = lo;
    const int q_len = a.cu_seqlens_q[seq + 1] - a.cu_seqlens_q[seq];
    limit = a.context_lens[seq] - q_len + (t - a.cu_seqlens_q[seq]);     // last visible key position
    total_pages = limit >= 0 ? limit / kPage + 1 : 0;
    bt = a.block_tables + (long long)seq * a.bt_stride;
  } else {
    total_pages = (a.topk + kPage - 1) / kPage;                           // tiles of 64 listed rows; the list is already causal
  }
  const int per_split = (total_pages + a.splits - 1) / a.splits;
  const int pg_begin = split * per_split;
  const int pg_end = min(total_pages, pg_begin + per_split);
  const int n_tiles = max(0, pg_end - pg_begin);
  const int* ids = kSparse ? a.sparse + (long long)t * a.topk : nullptr;

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 128;

  if (kSparse && (warp == 0 || warp >= 6)) {
    // Four gather warps (0, 6, 7, 8); each owns 16 of the 64 listed rows of every tile.  A row's 512 latent bytes are one
    // warp-wide cp.async (lane = 16-byte chunk, fully coalesced); the 64 rope bytes of 8 rows share another.  Destinations
    // follow the 128-byte / 64-byte swizzle the tensor-core descriptors expect.
    if (n_tiles > 0) {
      const int lane = (int)lane_id();
      const int pw = warp == 0 ? 0 : warp - 5;
      const int r_lo = pw * 16;
      if (warp == 0 && lane == 0) {
        const int qrow = t * a.H;
        mbar_expect_tx(b_qfull, kQBytes);
        for (int p = 0; p < 4; p++) tma_load_2d(smem_u32(sQ + p * 128 * 128), &tq128, b_qfull, p * 128, qrow);
        tma_load_2d(smem_u32(sQ + kQNope), &tq64, b_qfull, 512, qrow);
      }
      // listed row id of row r_lo + (lane & 15) of tile i; anything that is not a cache row becomes -1 (zero-filled, never read)
      auto load_id = [&](int i) -> int {
        const int k = (pg_begin + i) * kPage + r_lo + (lane & 15);
        int id = -1;
        if (i < n_tiles && k < a.topk) id = ids[k];
        return (id >= 0 && (long long)id < a.cache_rows) ? id : -1;
      };
      int id_next = load_id(0);
      // One cp.async group per iteration (empty once the tiles run out).  At the top of iteration i the groups 0 .. i-1 are
      // committed, so "all but the newest one have landed" means this lane's part of tile i-2 is complete: it is fenced for
      // the tensor-core proxy and handed over BEFORE the warp blocks on the slot tile i goes into - that slot is freed by the
      // product that runs after the scores of tile i-2, so handing over after the wait would deadlock.  Two tiles stay in
      // flight behind the one being consumed, and the ids of tile i+1 are fetched while tile i is issued.
      bool ok = true;
      for (int i = 0; i < n_tiles + 2; i++) {
        const int j = i - 2;
        if (j >= 0 && j < n_tiles) {
          cp_async_wait<1>();
          fence_proxy_async_smem();
          mbar_arrive(b_pgfull + 8 * (j % kPgStages));
        }
        if (i < n_tiles && ok) {
          const int s = i % kPgStages;
          ok = mbar_wait(b_pgempty + 8 * s, ((i / kPgStages) & 1) ^ 1, abort_flag, kKernelMla, 100 + s);
          ok = __all_sync(0xffffffffu, ok);
          if (ok) {
            const int my_id = id_next;
            id_next = load_id(i + 1);
            const uint32_t dst = smem_u32(sPg + s * kPgBytes);
            const uint32_t d_nope = dst + (lane >> 3) * (kPage * 128);
            const uint8_t* src_nope = a.cache + lane * 16;
#pragma unroll
            for (int r = 0; r < 16; r++) {
              const int row = r_lo + r;
              const int id = __shfl_sync(0xffffffffu, my_id, r);
              const bool valid = id >= 0;
              cp_async16(d_nope + row * 128 + (((lane & 7) ^ (row & 7)) << 4), src_nope + (valid ? (long long)id * kDk : 0), valid ? 16u : 0u);
            }
#pragma unroll
            for (int it = 0; it < 2; it++) {
              const int rr = it * 8 + (lane >> 2), row = r_lo + rr, ch = lane & 3;
              const int id = __shfl_sync(0xffffffffu, my_id, rr);
              const bool valid = id >= 0;
              cp_async16(dst + kPgNope + row * 64 + ((ch ^ ((row >> 1) & 3)) << 4),
                         a.cache + (valid ? (long long)id * kDk + kDv + ch * 16 : 0), valid ? 16u : 0u);
            }
          }
        }
        cp_async_commit();
      }
      cp_async_wait<0>();
    }
  } else if (warp == 0) {
    if (n_tiles > 0 && elect_one()) {
      const int qrow = t * a.H;
      mbar_expect_tx(b_qfull, kQBytes);
      for (int p = 0; p < 4; p++) tma_load_2d(smem_u32(sQ + p * 128 * 128), &tq128, b_qfull, p * 128, qrow);
      tma_load_2d(smem_u32(sQ + kQNope), &tq64, b_qfull, 512, qrow);
      for (int i = 0; i < n_tiles; i++) {
        const int s = i % kPgStages;
        if (!mbar_wait(b_pgempty + 8 * s, ((i / kPgStages) & 1) ^ 1, abort_flag, kKernelMla, 100 + s)) break;
        int block = bt[pg_begin + i];
        if (!NE_INDEX_OK(block, BK_CACHE_PAGES, kKernelMla, __LINE__)) block = 0;      // a bad page id reads page 0 instead of another allocation
        uint8_t* dst = sPg + s * kPgBytes;
        mbar_expect_tx(b_pgfull + 8 * s, kPgBytes);
        for (int p = 0; p < 4; p++) tma_load_3d(smem_u32(dst + p * kPage * 128), &tk128, b_pgfull + 8 * s, p * 128, 0, block);
        tma_load_3d(smem_u32(dst + kPgNope), &tk64, b_pgfull + 8 * s, 512, 0, block);
      }
    }
  } else if (warp == 1) {
    if (n_tiles > 0 && elect_one()) {
      constexpr uint32_t kIdescQK = make_idesc(FMT_E4M3, FMT_E4M3, 128, kPage);
      constexpr uint32_t kIdescPV = make_idesc(FMT_E4M3, FMT_E4M3, 128, kVHalf, 0, 1);   // B (= V) is MN-major
      bool ok = mbar_wait(b_qfull, 0, abort_flag, kKernelMla, 200);
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      auto pv = [&](int j) -> bool {
        if (!mbar_wait(b_pfull + 8 * (j & 1), (j >> 1) & 1, abort_flag, kKernelMla, 230)) return false;
        tc_fence_after();
        const int s = j % kPgStages;
        const uint32_t pg = smem_u32(sPg + s * kPgBytes);
#pragma unroll
        for (int ks = 0; ks < 2; ks++) {
          uint64_t adesc = make_smem_desc(p_addr + (j & 1) * kPBytes + ks * 32, 16, 512, SW_64B);
          uint64_t bdesc = make_smem_desc(pg + (vhalf * 2) * kPage * 128 + ks * 32 * 128, 8192, 1024, SW_128B);
          umma_f8(tmem_o, adesc, bdesc, kIdescPV, (j | ks) != 0);
        }
        tc_commit(b_pgempty + 8 * s);
        tc_commit(b_pempty + 8 * (j & 1));
        return true;
      };
      // An mbarrier test costs ~150 cycles even when the phase completed long ago and this thread is the serial resource of
      // the CTA, so the two barriers that gate S(i+1) are tested before the MMAs of P V(i-1) / S(i) are issued (issuing blocks
      // for about as long as the MMAs run); only a failed test falls back to waiting.
      bool pre_se = true, pre_pg = mbar_test(b_pgfull, 0);
      for (int i = 0; ok && i < n_tiles; i++) {
        const int sb = i & 1, s = i % kPgStages;
        if (!pre_se && !mbar_wait(b_sempty + 8 * sb, ((i >> 1) & 1) ^ 1, abort_flag, kKernelMla, 210 + sb)) { ok = false; break; }
        if (!pre_pg && !mbar_wait(b_pgfull + 8 * s, (i / kPgStages) & 1, abort_flag, kKernelMla, 220 + s)) { ok = false; break; }
        mbar_test2(b_sempty + 8 * ((i + 1) & 1), (((i + 1) >> 1) & 1) ^ 1, b_pgfull + 8 * ((i + 1) % kPgStages), ((i + 1) / kPgStages) & 1,
                   pre_se, pre_pg);
        tc_fence_after();
        const uint32_t pg = smem_u32(sPg + s * kPgBytes);
        const uint32_t d = tmem_base + sb * kPage;
#pragma unroll
        for (int p = 0; p < 4; p++) {
#pragma unroll
          for (int ks = 0; ks < 4; ks++) {
            uint64_t adesc = make_smem_desc(q_addr + p * 128 * 128 + ks * 32, 16, 1024, SW_128B);
            uint64_t bdesc = make_smem_desc(pg + p * kPage * 128 + ks * 32, 16, 1024, SW_128B);
            umma_f8(d, adesc, bdesc, kIdescQK, (p | ks) != 0);
          }
        }
#pragma unroll
        for (int ks = 0; ks < 2; ks++) {
          uint64_t adesc = make_smem_desc(q_addr + kQNope + ks * 32, 16, 512, SW_64B);
          uint64_t bdesc = make_smem_desc(pg + kPgNope + ks * 32, 16, 512, SW_64B);
          umma_f8(d, adesc, bdesc, kIdescQK, 1);
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
    const bool row_ok = row < a.H;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    bool s_ready = false;                            // early test of the next page's S buffer (see below)
    for (int i = 0; ok && i < n_tiles; i++) {
      const int sb = i & 1;
      const int key0 = (pg_begin + i) * kPage;
      bool in_lo = true, in_hi = true;               // sparse: is the listed row a cache row (fetched before the wait, used after)
      if (kSparse) {
        const int l = key0 + (int)lane_id();
        const int id_lo = l < a.topk ? ids[l] : -1, id_hi = l + 32 < a.topk ? ids[l + 32] : -1;
        in_lo = id_lo >= 0 && (long long)id_lo < a.cache_rows;
        in_hi = id_hi >= 0 && (long long)id_hi < a.cache_rows;
      }
      if (!s_ready && !mbar_wait(b_sfull + 8 * sb, (i >> 1) & 1, abort_flag, kKernelMla, 300 + sb)) { ok = false; break; }
      tc_fence_after();
      uint32_t r0[32], r1[32];
      tmem_ld_32x32b_x32(tmem_base + lane_addr + sb * kPage, r0);
      tmem_ld_32x32b_x32(tmem_base + lane_addr + sb * kPage + 32, r1);
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane_id() == 0) mbar_arrive(b_sempty + 8 * sb);
      // this page's P buffer was last read by the P V product of page i-2: tested here, long before the answer is needed
      // (an mbarrier test costs ~150 cycles even when the phase completed long ago)
      const bool p_free = i < 2 || mbar_test(b_pempty + 8 * (i & 1), ((i - 2) >> 1) & 1);
      if (kSparse) {
        // columns whose listed row id is not a cache row (-1, or past the list) hold zero-filled keys: take them out of the softmax
        const unsigned v_lo = __ballot_sync(0xffffffffu, in_lo), v_hi = __ballot_sync(0xffffffffu, in_hi);
        if (!row_ok || (v_lo & v_hi) != 0xffffffffu) {
#pragma unroll
          for (int j = 0; j < 32; j++) {
            if (!row_ok || !((v_lo >> j) & 1u)) r0[j] = 0xff800000u;
            if (!row_ok || !((v_hi >> j) & 1u)) r1[j] = 0xff800000u;
          }
        }
      } else if (!row_ok || key0 + kPage - 1 > limit) {                 // only the page that straddles the causal limit needs masking
#pragma unroll
        for (int j = 0; j < 32; j++) {
          if (!row_ok || key0 + j > limit) r0[j] = 0xff800000u;
          if (!row_ok || key0 + 32 + j > limit) r1[j] = 0xff800000u;
        }
      }
      // four independent chains for the maximum; the (positive) scale is applied once at the end
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        mx[0] = fmaxf(mx[0], __uint_as_float(r0[j])); mx[1] = fmaxf(mx[1], __uint_as_float(r0[j + 1]));
        mx[2] = fmaxf(mx[2], __uint_as_float(r1[j])); mx[3] = fmaxf(mx[3], __uint_as_float(r1[j + 1]));
      }
      const float m_tile = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * a.scale_log2;
      // Lazy rescaling: the reference maximum only moves when the page's maximum exceeds it by more than 2^8.  Until then
      // probabilities may be as large as 256 (inside e4m3's range, same relative precision) and O needs no correction;
      // the result is exact because l_run is accumulated against the same reference.
      const bool first_valid = (m_run == -INFINITY);
      const float m_new = (first_valid || m_tile > m_run + 8.f) ? fmaxf(m_run, m_tile) : m_run;
      const float alpha = (m_new == -INFINITY || first_valid) ? 1.f : exp2f(m_run - m_new);
      const float neg_m = (m_new == -INFINITY) ? 0.f : -m_new;      // masked scores are -inf and come out as 0 either way
      float ps[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t pk[16];
#pragma unroll
      for (int j = 0; j < 8; j++) {
        const float p0 = exp2f(fmaf(__uint_as_float(r0[4 * j]), a.scale_log2, neg_m)), p1 = exp2f(fmaf(__uint_as_float(r0[4 * j + 1]), a.scale_log2, neg_m));
        const float p2 = exp2f(fmaf(__uint_as_float(r0[4 * j + 2]), a.scale_log2, neg_m)), p3 = exp2f(fmaf(__uint_as_float(r0[4 * j + 3]), a.scale_log2, neg_m));
        const float q0 = exp2f(fmaf(__uint_as_float(r1[4 * j]), a.scale_log2, neg_m)), q1 = exp2f(fmaf(__uint_as_float(r1[4 * j + 1]), a.scale_log2, neg_m));
        const float q2 = exp2f(fmaf(__uint_as_float(r1[4 * j + 2]), a.scale_log2, neg_m)), q3 = exp2f(fmaf(__uint_as_float(r1[4 * j + 3]), a.scale_log2, neg_m));
        ps[0] += p0 + p1; ps[1] += p2 + p3; ps[2] += q0 + q1; ps[3] += q2 + q3;
        pk[j] = pack_e4m3x4(p0, p1, p2, p3);
        pk[8 + j] = pack_e4m3x4(q0, q1, q2, q3);
      }
      l_run = l_run * alpha + ((ps[0] + ps[1]) + (ps[2] + ps[3]));
      m_run = m_new;
      // O may only be rescaled once the previous page's P V product has retired; that is rare with lazy rescaling
      if (i > 0 && __any_sync(0xffffffffu, alpha < 1.f)) {
        if (!mbar_wait(b_pempty + 8 * ((i - 1) & 1), ((i - 1) >> 1) & 1, abort_flag, kKernelMla, 310)) { ok = false; break; }
        tc_fence_after();
#pragma unroll 1
        for (int cblk = 0; cblk < kVHalf / 16; cblk++) {
          uint32_t o[16];
          tmem_ld_32x32b_x16(tmem_o + lane_addr + cblk * 16, o);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; j++) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
          tmem_st_32x32b_x16(tmem_o + lane_addr + cblk * 16, o);
        }
        tc_wait_st();
      }
      // this page's P buffer was last read by the P V product of page i-2
      if (!p_free && !mbar_wait(b_pempty + 8 * (i & 1), ((i - 2) >> 1) & 1, abort_flag, kKernelMla, 311)) { ok = false; break; }
      // S of the next page is usually complete by now: test it before the stores so the answer is there at the loop top
      s_ready = mbar_test(b_sfull + 8 * ((i + 1) & 1), ((i + 1) >> 1) & 1);
      // P row (64 e4m3 = 4 chunks of 16 bytes) into the 64B-swizzled K-major layout the MMA reads
      {
        uint8_t* prow = sP + (i & 1) * kPBytes + row * 64;
        const int sw = (row >> 1) & 3;
#pragma unroll
        for (int cch = 0; cch < 4; cch++)
          *reinterpret_cast<uint4*>(prow + ((cch ^ sw) << 4)) = make_uint4(pk[4 * cch], pk[4 * cch + 1], pk[4 * cch + 2], pk[4 * cch + 3]);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane_id() == 0) mbar_arrive(b_pfull + 8 * (i & 1));
    }
    if (ok && n_tiles > 0) ok = mbar_wait(b_pempty + 8 * ((n_tiles - 1) & 1), ((n_tiles - 1) >> 1) & 1, abort_flag, kKernelMla, 320);
    if (ok && n_tiles > 0) {
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      const long long orow = (long long)t * a.H + row;
#pragma unroll 1
      for (int cblk = 0; cblk < kVHalf / 32; cblk++) {
        uint32_t o[32];
        tmem_ld_32x32b_x32(tmem_o + lane_addr + cblk * 32, o);
        tc_wait_ld();
        if (row_ok) {
          if (a.splits == 1) {
            __nv_bfloat16* dst = a.out + orow * kDv + vhalf * kVHalf + cblk * 32;
#pragma unroll
            for (int v = 0; v < 4; v++) {
              *reinterpret_cast<uint4*>(dst + v * 8) = make_uint4(
                  pack_bf16x2(__uint_as_float(o[v * 8]) * inv, __uint_as_float(o[v * 8 + 1]) * inv),
                  pack_bf16x2(__uint_as_float(o[v * 8 + 2]) * inv, __uint_as_float(o[v * 8 + 3]) * inv),
                  pack_bf16x2(__uint_as_float(o[v * 8 + 4]) * inv, __uint_as_float(o[v * 8 + 5]) * inv),
                  pack_bf16x2(__uint_as_float(o[v * 8 + 6]) * inv, __uint_as_float(o[v * 8 + 7]) * inv));
            }
          } else {
            float* dst = a.part + ((long long)split * a.T * a.H + orow) * kDv + vhalf * kVHalf + cblk * 32;
#pragma unroll
            for (int v = 0; v < 8; v++)
              *reinterpret_cast<float4*>(dst + v * 4) = make_float4(__uint_as_float(o[v * 4]) * inv, __uint_as_float(o[v * 4 + 1]) * inv,
                                                                    __uint_as_float(o[v * 4 + 2]) * inv, __uint_as_float(o[v * 4 + 3]) * inv);
          }
        }
      }
    }
    if (a.splits > 1 && vhalf == 0 && row_ok)
      a.lse2[(long long)split * a.T * a.H + (long long)t * a.H + row] = (ok && l_run > 0.f) ? m_run + log2f(l_run) : -INFINITY;
    if (a.splits == 1 && n_tiles == 0 && row_ok) {
      // a token that sees no key (cannot happen for causal self-attention, kept for safety): zero output
      __nv_bfloat16* dst = a.out + ((long long)t * a.H + row) * kDv + vhalf * kVHalf;
      for (int cidx = 0; cidx < kVHalf; cidx += 8) *reinterpret_cast<uint4*>(dst + cidx) = make_uint4(0, 0, 0, 0);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) for (int i = 0; i < 2000; i++) __nanosleep(1000);
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// bf16 -> e4m3 with clamp, no scale (queries of the fp8 attention path)
__global__ void cast_e4m3_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ y, long long n) {
  long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= n) return;
  uint4 v = *reinterpret_cast<const uint4*>(x + i);
  float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
  *reinterpret_cast<uint2*>(y + i) = make_uint2(pack_e4m3x4(a.x, a.y, b.x, b.y), pack_e4m3x4(c.x, c.y, d.x, d.y));
}

}  // namespace ne

using namespace ne;

extern "C" int ne_cast_e4m3(const void* x, void* y, long long n, cudaStream_t st) {
  if (n <= 0) return 0;
  if (n % 8) return 1001;
  cast_e4m3_kernel<<<(unsigned)((n / 8 + 255) / 256), 256, 0, st>>>((const __nv_bfloat16*)x, (uint8_t*)y, n);
  return (int)cudaGetLastError();
}

// q8 [T*H, 576] e4m3 (contiguous), cache [num_blocks, 64, 576] e4m3.  out bf16 [T, H, 512] when splits == 1, otherwise
// part fp32 [splits, T, H, 512] + lse2 fp32 [splits, T, H] for ne_attn_merge.
extern "C" int ne_mla_fp8(const void* q8, const void* cache, int num_blocks, const int* block_tables, int bt_stride,
                          const int* cu_seqlens_q, const int* context_lens, int num_seqs, int T, int H, int splits, float scale,
                          void* out, float* part, float* lse2, cudaStream_t st) {
  if (T <= 0) return 0;
  if (H > 128 || H < 1 || splits < 1 || (splits > 1 && (!part || !lse2))) return 1001;
  CUtensorMap tq128, tq64, tk128, tk64;
  {
    uint64_t dims[2] = {(uint64_t)kDk, (uint64_t)T * H}; uint64_t strides[1] = {(uint64_t)kDk};
    uint32_t b128[2] = {128, 128}, b64[2] = {64, 128};
    int rc = make_tmap(&tq128, q8, TMA_U8, 2, dims, strides, b128, TMA_SW_128); if (rc) return 2000 + rc;
    rc = make_tmap(&tq64, q8, TMA_U8, 2, dims, strides, b64, TMA_SW_64); if (rc) return 2100 + rc;
  }
  {
    uint64_t dims[3] = {(uint64_t)kDk, (uint64_t)kPage, (uint64_t)num_blocks}; uint64_t strides[2] = {(uint64_t)kDk, (uint64_t)kDk * kPage};
    uint32_t b128[3] = {128, kPage, 1}, b64[3] = {64, kPage, 1};
    int rc = make_tmap(&tk128, cache, TMA_U8, 3, dims, strides, b128, TMA_SW_128); if (rc) return 2200 + rc;
    rc = make_tmap(&tk64, cache, TMA_U8, 3, dims, strides, b64, TMA_SW_64); if (rc) return 2300 + rc;
  }
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(mla_fp8_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMlaSmem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  MlaArgs a;
  a.block_tables = block_tables; a.bt_stride = bt_stride; a.cu_seqlens_q = cu_seqlens_q; a.context_lens = context_lens; a.num_seqs = num_seqs;
  a.T = T; a.H = H; a.splits = splits; a.scale_log2 = scale * 1.4426950408889634f; a.out = (__nv_bfloat16*)out; a.part = part; a.lse2 = lse2;
  a.sparse = nullptr; a.topk = 0; a.cache = nullptr; a.cache_rows = 0;
  dim3 grid(2 * T, splits, 1);
  return (int)launch_pdl(mla_fp8_kernel<false>, grid, dim3(kMlaThreads), kMlaSmem, st, tq128, tq64, tk128, tk64, a);
}

// Sparse form: every query token attends the `topk` cache rows listed for it (sparse int32 [T, topk], row id = block * 64 +
// offset, -1 = none; the list must already respect causality).  Same outputs as ne_mla_fp8.
extern "C" int ne_mla_fp8_sparse(const void* q8, const void* cache, int num_blocks, const int* sparse, int topk, int T, int H, int splits,
                                 float scale, void* out, float* part, float* lse2, cudaStream_t st) {
  if (T <= 0) return 0;
  if (H > 128 || H < 1 || splits < 1 || topk < 1 || !sparse || (splits > 1 && (!part || !lse2))) return 1001;
  CUtensorMap tq128, tq64;
  {
    uint64_t dims[2] = {(uint64_t)kDk, (uint64_t)T * H}; uint64_t strides[1] = {(uint64_t)kDk};
    uint32_t b128[2] = {128, 128}, b64[2] = {64, 128};
    int rc = make_tmap(&tq128, q8, TMA_U8, 2, dims, strides, b128, TMA_SW_128); if (rc) return 2000 + rc;
    rc = make_tmap(&tq64, q8, TMA_U8, 2, dims, strides, b64, TMA_SW_64); if (rc) return 2100 + rc;
  }
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(mla_fp8_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMlaSmem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  MlaArgs a;
  a.block_tables = nullptr; a.bt_stride = 0; a.cu_seqlens_q = nullptr; a.context_lens = nullptr; a.num_seqs = 0;
  a.T = T; a.H = H; a.splits = splits; a.scale_log2 = scale * 1.4426950408889634f; a.out = (__nv_bfloat16*)out; a.part = part; a.lse2 = lse2;
  a.sparse = sparse; a.topk = topk; a.cache = (const uint8_t*)cache; a.cache_rows = (long long)num_blocks * kPage;
  dim3 grid(2 * T, splits, 1);
  return (int)launch_pdl(mla_fp8_kernel<true>, grid, dim3(kMlaSparseThreads), kMlaSmem, st, tq128, tq64, tq128, tq64, a);     // the key maps are unused here
}

// ---- allocation-free entry point ----------------------------------------------------------------------
// (declared in ne_noalloc.h; this entry point has no counterpart in the reference)
//
// Split-KV decode needs scratch for the per-slice partial outputs and their log-sum-exp values.  The regular entry point
// takes that scratch from its caller.  Some callers have nowhere to get it: a C host program that links this library
// without a tensor allocator, or code that runs where cudaMalloc is not allowed (inside a stream capture, or in a process
// whose memory was carved up front).  For them the scratch lives in a file-scope device array of fixed size, so every GPU
// that loads the library carries kNoAllocScratchBytes of it until the process exits.
namespace ne {
constexpr long long kNoAllocMaxSliceRows = 4096;                                  // splits * T * H may not exceed this
constexpr long long kNoAllocScratchBytes = kNoAllocMaxSliceRows * (kDv + 1) * 4;  // partial outputs + log-sum-exp, fp32
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];
}  // namespace ne

extern "C" int ne_attn_merge(const float* part, const float* lse2, void* out, int splits, long long rows, int D, int out_row_stride, cudaStream_t st);

// Same contract as ne_mla_fp8 with splits >= 1, but the caller passes inputs and the output only.
// * The first call on a device resolves the device address of the scratch array (cudaGetSymbolAddress) for that device;
//   make that first call outside any stream capture.  The address is cached per device.
// * Nothing in the scratch has to start at zero: every (slice, row) the merge reads is written by the attention kernel of
//   the same call, and slices that saw no key are marked by an infinite log-sum-exp and skipped.
// * All calls on a device share the one array.  Calls that may overlap on the GPU (different streams without an ordering
//   between them) race on it; issue them on one stream or order them with events.
// * Returns 1101 when splits * T * H exceeds kNoAllocMaxSliceRows (4096); no cudaMalloc / cudaFree is made on any path.
extern "C" int ne_mla_fp8_noalloc(const void* q8, const void* cache, int num_blocks, const int* block_tables, int bt_stride,
                                  const int* cu_seqlens_q, const int* context_lens, int num_seqs, int T, int H, int splits, float scale,
                                  void* out, cudaStream_t st) {
  // per-device address of the scratch array; atomics because host threads may make their first calls at the same time
  // (they would all resolve the same address, so the last store wins harmlessly)
  static std::atomic<unsigned char*> scratch_of_device[64];
  if (T <= 0) return 0;
  if (splits < 1 || H < 1 || H > 128) return 1001;
  const long long slice_rows = (long long)splits * T * H;
  if (slice_rows > kNoAllocMaxSliceRows) return 1101;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return 1102;
  unsigned char* scratch = scratch_of_device[dev].load(std::memory_order_acquire);
  if (!scratch) {
    // in host code the array's name is only a handle; the kernels need its address in this device's memory
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    scratch = static_cast<unsigned char*>(p);
    scratch_of_device[dev].store(scratch, std::memory_order_release);
  }
  if (splits == 1)
    return ne_mla_fp8(q8, cache, num_blocks, block_tables, bt_stride, cu_seqlens_q, context_lens, num_seqs, T, H, 1, scale, out, nullptr, nullptr, st);
  float* part = reinterpret_cast<float*>(scratch);
  float* lse2 = part + slice_rows * kDv;
  int rc = ne_mla_fp8(q8, cache, num_blocks, block_tables, bt_stride, cu_seqlens_q, context_lens, num_seqs, T, H, splits, scale, out, part, lse2, st);
  if (rc) return rc;
  return ne_attn_merge(part, lse2, out, splits, (long long)T * H, kDv, kDv, st);
}
