// tcgen05 GEMM family for sm_100a:  D[g, m, n] = sum_k A[g, m, k] * B[g, n, k]   (both operands K-major).
//
//  * bf16 x bf16 -> fp32 accumulation in TMEM, bf16 or fp32 output
//  * fp8 e4m3 x e4m3 with DeepSeek block scales (activations 1x128, weights 128x128): each 128-deep K block is
//    multiplied on the tensor cores into a fresh TMEM accumulator and promoted into fp32 registers with
//    scale_a[m, kb] * scale_b[n/128, kb] by the epilogue warps while the next K block is being multiplied
//  * dense (one group, M rows) or grouped-masked (E groups of up to max_m rows, masked_m[e] valid), the layout
//    the MoE path uses for prefill and decode alike
//
// Structure (one CTA per SM, persistent over tiles): warp 0 issues TMA loads into a multi-stage 128B-swizzled
// shared-memory ring, warp 1 issues tcgen05.mma from one elected thread and owns the TMEM allocation, warps 2-5
// drain TMEM (tcgen05.ld), apply scales, convert and store.  Two TMEM accumulators let the epilogue of one tile
// (or K block) overlap the MMAs of the next.  All mbarrier waits are bounded.
//
// Replaces in the reference: deep_gemm.fp8_gemm_nt / m_grouped_fp8_gemm_nt_masked call sites
// (layers/backends/linear/deep_gemm.py, layers/backends/experts/deep_gemm.py:498-837), the CuTe-DSL small-M bf16
// GEMM (kernel/cutedsl_bf16_gemm.py) and cuBLAS F.linear (layers/backends/linear/generic.py:103-315).
#include <mutex>
#include <unordered_map>

#include "ptx.cuh"
#include "tma_host.h"

namespace ne {

__device__ int g_status[8];

constexpr int kBlockM = 128;
constexpr int kKBytes = 128;            // bytes of K per stage row: one 128B swizzle atom
constexpr int kGemmThreads = 192;
constexpr int kKernelGemm = 1;

struct GemmArgs {
  int M, N, K, groups;
  const int* masked_m;                  // [groups] valid rows per group, or nullptr (all M rows valid)
  const int* row_start;                 // contiguous mode: group g owns rows [row_start[g], row_start[g] + masked_m[g]) of one
                                        // flat [M, K] activation matrix (starts are multiples of 128); nullptr = [groups, M, K]
  int a_group_inner;                    // A is stored [rows, groups, K]: TMA coordinates are (k, group, row)
  void* D; long long ldd; long long d_group_stride;   // in elements
  const float* sa; int sa_ld; long long sa_group_stride;   // activation scales [groups][K/128][sa_ld]
  const float* sb; long long sb_group_stride;              // weight scales [groups][ceil(N/128)][K/128]
  int out_fp32;
  const long long* row_dst;             // optional scatter epilogue: absolute address of every output row (bf16, may be peer memory),
  long long rd_group_stride;            // indexed [group * rd_group_stride + row]; used by the MoE combine
};

template <int BLOCK_N> struct Smem {
  static constexpr int kABytes = kBlockM * kKBytes;
  static constexpr int kBBytes = BLOCK_N * kKBytes;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStaging = 8 * 32 * 80;      // per-warp epilogue staging for up to 8 epilogue warps
  static constexpr int kBudget = 232448 - 1024 - 256 - kStaging;
  static constexpr int kStages = (kBudget / kStageBytes) > 10 ? 10 : (kBudget / kStageBytes);
  static constexpr int kBytes = kStages * kStageBytes + kStaging + 1024 /*align*/ + 256 /*barriers*/;
};

struct TileSched {
  int groups, M, n_blocks;
  const int* masked_m;
  const int* row_start;
  int g = 0, base = 0;
  __device__ TileSched(int groups_, int M_, int nb, const int* mm, const int* rs) : groups(groups_), M(M_), n_blocks(nb), masked_m(mm), row_start(rs) {}
  __device__ int row0(int grp) const { return row_start ? row_start[grp] : 0; }
  __device__ int rows(int grp) const {
    int r = masked_m ? masked_m[grp] : M;
    int cap = row_start ? M - row_start[grp] : M;      // never step outside the buffer, whatever the counts say
    return r < cap ? r : (cap > 0 ? cap : 0);
  }
  __device__ bool get(int tile, int& grp, int& mb, int& nb) {
    while (g < groups) {
      int cnt = ((rows(g) + kBlockM - 1) / kBlockM) * n_blocks;
      if (tile < base + cnt) { int l = tile - base; grp = g; mb = l / n_blocks; nb = l % n_blocks; return true; }
      base += cnt; g++;
    }
    return false;
  }
};

// bf16 output goes through a small per-warp staging buffer: each thread parks 32 columns of its row (64 bytes), then the
// warp writes eight rows per instruction with four lanes covering each row's 64 contiguous bytes.  Compared with every
// thread writing 16 bytes of a different row this quadruples the contiguous run per row - what matters most when the rows
// are scattered to peer GPUs by the MoE combine.
constexpr int kStgPitch = 80;                       // 64 bytes of data + 16 of padding: conflict-free for 16-byte accesses
constexpr int kStgWarpBytes = 32 * kStgPitch;
__device__ __forceinline__ void epi_store32_bf16(uint8_t* stg, const float (&v)[32], bool row_ok, __nv_bfloat16* drow, int ncols_left) {
  const int lane = (int)lane_id();
  uint8_t* mine = stg + lane * kStgPitch;
#pragma unroll
  for (int q = 0; q < 4; q++)
    *reinterpret_cast<uint4*>(mine + q * 16) = make_uint4(pack_bf16x2(v[q * 8], v[q * 8 + 1]), pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]),
                                                          pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]), pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]));
  __syncwarp();
  const int ch = lane & 3;
#pragma unroll
  for (int r0 = 0; r0 < 32; r0 += 8) {
    const int rr = r0 + (lane >> 2);
    const bool okr = __shfl_sync(0xffffffffu, (int)row_ok, rr) != 0;
    const unsigned long long dp = __shfl_sync(0xffffffffu, (unsigned long long)reinterpret_cast<uintptr_t>(drow), rr);
    if (okr && ch * 8 < ncols_left)
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(dp) + ch * 8) = *reinterpret_cast<const uint4*>(stg + rr * kStgPitch + ch * 16);
  }
  __syncwarp();
}

// Block-scaled tiles at least 64 wide use two epilogue warpgroups that split the tile's columns, halving the
// promotion work per thread and per K block.
template <int BLOCK_N, bool kBlockScaled> struct EpiCfg {
  static constexpr int kGroups = (kBlockScaled && BLOCK_N >= 64) ? 2 : 1;
  static constexpr int kThreads = 64 + 128 * kGroups;
};

template <int BLOCK_N, bool kFP8, bool kBlockScaled>
__global__ void __launch_bounds__((EpiCfg<BLOCK_N, kBlockScaled>::kThreads), 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const GemmArgs args) {
  using S = Smem<BLOCK_N>;
  constexpr int kStages = S::kStages;
  constexpr int kElemsPerStageK = kFP8 ? 128 : 64;
  constexpr int kUmmaK = kFP8 ? 32 : 16;
  constexpr int kMmasPerStage = kElemsPerStageK / kUmmaK;     // 4
  // TMEM accumulator ring: block-scaled GEMMs hand one accumulator per K block to the epilogue, so they use the
  // deepest ring 512 columns allow (up to 4); plain GEMMs hand over one per tile and need two.
  constexpr int kAcc = kBlockScaled ? ((512 / BLOCK_N) > 4 ? 4 : (512 / BLOCK_N)) : 2;
  constexpr uint32_t kTmemCols = (kAcc * BLOCK_N) < 32 ? 32 : kAcc * BLOCK_N;
  constexpr uint32_t kIdesc = make_idesc(kFP8 ? FMT_E4M3 : FMT_BF16, kFP8 ? FMT_E4M3 : FMT_BF16, kBlockM, BLOCK_N);
  constexpr int kEpi = EpiCfg<BLOCK_N, kBlockScaled>::kGroups;
  constexpr int kCols = BLOCK_N / kEpi;          // columns of the tile each epilogue thread owns

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + kStages * S::kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + S::kStaging);
  // bars: full[kStages], empty[kStages], tmem_full[kAcc], tmem_empty[kAcc]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 2 * kAcc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + kStages);
  const uint32_t tfull0 = smem_u32(bars + 2 * kStages), tempty0 = smem_u32(bars + 2 * kStages + kAcc);
  const uint32_t smem_base = smem_u32(smem);

  const int warp = threadIdx.x >> 5;
  const int num_kb = (args.K + kElemsPerStageK - 1) / kElemsPerStageK;
  const int n_blocks = (args.N + BLOCK_N - 1) / BLOCK_N;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; i++) { mbar_init(full0 + 8 * i, 1); mbar_init(empty0 + 8 * i, 1); }
    for (int i = 0; i < kAcc; i++) { mbar_init(tfull0 + 8 * i, 1); mbar_init(tempty0 + 8 * i, 4 * kEpi); }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a); tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (elect_one()) {
      TileSched sched(args.groups, args.M, n_blocks, args.masked_m, args.row_start);
      int stage = 0; uint32_t phase = 0; int grp, mb, nb;
      bool ok = true;
      for (int tile = blockIdx.x; ok && sched.get(tile, grp, mb, nb); tile += gridDim.x) {
        for (int kb = 0; kb < num_kb; kb++) {
          if (!mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag, kKernelGemm, 100 + stage)) { ok = false; break; }
          uint32_t a_dst = smem_base + stage * S::kStageBytes, b_dst = a_dst + S::kABytes;
          mbar_expect_tx(full0 + 8 * stage, S::kStageBytes);
          if (args.a_group_inner) tma_load_3d(a_dst, &tmap_a, full0 + 8 * stage, kb * kElemsPerStageK, grp, mb * kBlockM);
          else tma_load_3d(a_dst, &tmap_a, full0 + 8 * stage, kb * kElemsPerStageK, sched.row0(grp) + mb * kBlockM, args.row_start ? 0 : grp);
          tma_load_3d(b_dst, &tmap_b, full0 + 8 * stage, kb * kElemsPerStageK, nb * BLOCK_N, grp);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (elect_one()) {
      TileSched sched(args.groups, args.M, n_blocks, args.masked_m, args.row_start);
      int stage = 0; uint32_t phase = 0; int buf = 0; uint32_t bphase = 0; int grp, mb, nb;
      bool ok = true;
      for (int tile = blockIdx.x; ok && sched.get(tile, grp, mb, nb); tile += gridDim.x) {
        if (!kBlockScaled) {
          if (!mbar_wait(tempty0 + 8 * buf, bphase ^ 1, abort_flag, kKernelGemm, 200 + buf)) { ok = false; break; }
          tc_fence_after();
        }
        for (int kb = 0; kb < num_kb; kb++) {
          if (kBlockScaled) {
            if (!mbar_wait(tempty0 + 8 * buf, bphase ^ 1, abort_flag, kKernelGemm, 210 + buf)) { ok = false; break; }
          }
          if (!mbar_wait(full0 + 8 * stage, phase, abort_flag, kKernelGemm, 300 + stage)) { ok = false; break; }
          tc_fence_after();
          uint32_t a_addr = smem_base + stage * S::kStageBytes, b_addr = a_addr + S::kABytes;
          uint64_t adesc = make_smem_desc(a_addr, 16, 1024, SW_128B);
          uint64_t bdesc = make_smem_desc(b_addr, 16, 1024, SW_128B);
          uint32_t d = tmem_base + buf * BLOCK_N;
#pragma unroll
          for (int k = 0; k < kMmasPerStage; k++) {
            uint32_t acc = kBlockScaled ? (k != 0) : ((kb | k) != 0);
            // advancing 32 bytes along K inside the 128B swizzle atom = +2 in the descriptor's 16-byte address units
            if (kFP8) umma_f8(d, adesc + 2 * k, bdesc + 2 * k, kIdesc, acc);
            else umma_f16(d, adesc + 2 * k, bdesc + 2 * k, kIdesc, acc);
          }
          tc_commit(empty0 + 8 * stage);                // smem slot reusable once these MMAs retire
          if (kBlockScaled) { tc_commit(tfull0 + 8 * buf); if (++buf == kAcc) { buf = 0; bphase ^= 1; } }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        if (!kBlockScaled) { tc_commit(tfull0 + 8 * buf); if (++buf == kAcc) { buf = 0; bphase ^= 1; } }
      }
    }
  } else {
    // ---------------- epilogue: 4 warps per group, warp w may touch TMEM lanes [32*(w%4), +32) ----------------
    const int wq = warp & 3;
    const int cbase = ((warp - 2) >> 2) * kCols;   // column offset of this warp's group inside the tile
    const int row_in_tile = wq * 32 + (int)lane_id();
    const uint32_t lane_addr = (uint32_t)(wq * 32) << 16;
    TileSched sched(args.groups, args.M, n_blocks, args.masked_m, args.row_start);
    int buf = 0; uint32_t bphase = 0; int grp, mb, nb;
    bool ok = true;
    for (int tile = blockIdx.x; ok && sched.get(tile, grp, mb, nb); tile += gridDim.x) {
      const bool row_ok = mb * kBlockM + row_in_tile < sched.rows(grp);
      const int row = sched.row0(grp) + mb * kBlockM + row_in_tile;      // row inside the group's (or the flat) matrix
      const int n0 = nb * BLOCK_N;
      if (kBlockScaled) {
        float acc[kCols];
#pragma unroll
        for (int j = 0; j < kCols; j++) acc[j] = 0.f;
        const float* sa = args.sa + (long long)grp * args.sa_group_stride + (row_ok ? row : 0);
        const float* sb = args.sb + (long long)grp * args.sb_group_stride + (long long)(n0 / 128) * num_kb;
        // scale factors are fetched four K blocks ahead so their L2 latency hides behind the promotion work
        constexpr int kPf = 4;
        float nxt[kPf];
#pragma unroll
        for (int j = 0; j < kPf; j++) nxt[j] = j < num_kb ? __ldg(sa + (long long)j * args.sa_ld) * __ldg(sb + j) : 0.f;
        for (int kb0 = 0; kb0 < num_kb && ok; kb0 += kPf) {
          float cur[kPf];
#pragma unroll
          for (int j = 0; j < kPf; j++) {
            cur[j] = nxt[j];
            const int kn = kb0 + kPf + j;
            nxt[j] = kn < num_kb ? __ldg(sa + (long long)kn * args.sa_ld) * __ldg(sb + kn) : 0.f;
          }
#pragma unroll
        for (int jj = 0; jj < kPf; jj++) {
          if (kb0 + jj >= num_kb || !ok) break;
          const float s = cur[jj];
          if (!mbar_wait(tfull0 + 8 * buf, bphase, abort_flag, kKernelGemm, 400 + buf)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < kCols / 32; c += 2) {
            // two TMEM loads in flight per wait
            uint32_t r0[32], r1[32];
            tmem_ld_32x32b_x32(tmem_base + lane_addr + buf * BLOCK_N + cbase + c * 32, r0);
            if (c + 1 < kCols / 32) tmem_ld_32x32b_x32(tmem_base + lane_addr + buf * BLOCK_N + cbase + (c + 1) * 32, r1);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; j++) acc[c * 32 + j] = fmaf(s, __uint_as_float(r0[j]), acc[c * 32 + j]);
            if (c + 1 < kCols / 32) {
#pragma unroll
              for (int j = 0; j < 32; j++) acc[(c + 1) * 32 + j] = fmaf(s, __uint_as_float(r1[j]), acc[(c + 1) * 32 + j]);
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane_id() == 0) mbar_arrive(tempty0 + 8 * buf);
          if (++buf == kAcc) { buf = 0; bphase ^= 1; }
        }
        }
        if (!ok) break;
        {
          const long long off = (long long)grp * args.d_group_stride + (long long)row * args.ldd + n0 + cbase;
          if (args.out_fp32) {
            if (row_ok) {
#pragma unroll
              for (int c = 0; c < kCols / 8; c++) {
                if (n0 + cbase + c * 8 < args.N) {
                  float4* p = reinterpret_cast<float4*>(reinterpret_cast<float*>(args.D) + off + c * 8);
                  p[0] = make_float4(acc[c * 8], acc[c * 8 + 1], acc[c * 8 + 2], acc[c * 8 + 3]);
                  p[1] = make_float4(acc[c * 8 + 4], acc[c * 8 + 5], acc[c * 8 + 6], acc[c * 8 + 7]);
                }
              }
            }
          } else {
            __nv_bfloat16* dbf = (args.row_dst && row_ok)
                ? reinterpret_cast<__nv_bfloat16*>(args.row_dst[(long long)grp * args.rd_group_stride + row]) + n0 + cbase
                : reinterpret_cast<__nv_bfloat16*>(args.D) + off;
            uint8_t* stg = staging + (warp - 2) * kStgWarpBytes;
#pragma unroll
            for (int cc = 0; cc < kCols / 32; cc++) {
              float v[32];
#pragma unroll
              for (int j = 0; j < 32; j++) v[j] = acc[cc * 32 + j];
              epi_store32_bf16(stg, v, row_ok, dbf + cc * 32, args.N - (n0 + cbase + cc * 32));
            }
          }
        }
      } else {
        if (!mbar_wait(tfull0 + 8 * buf, bphase, abort_flag, kKernelGemm, 410 + buf)) { ok = false; break; }
        tc_fence_after();
        long long off = (long long)grp * args.d_group_stride + (long long)row * args.ldd + n0;
        __nv_bfloat16* dbf = (args.row_dst && row_ok) ? reinterpret_cast<__nv_bfloat16*>(args.row_dst[(long long)grp * args.rd_group_stride + row]) + n0
                                                      : reinterpret_cast<__nv_bfloat16*>(args.D) + off;
#pragma unroll
        for (int c = 0; c < BLOCK_N / 32; c++) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem_base + lane_addr + buf * BLOCK_N + c * 32, r);
          tc_wait_ld();
          if (args.out_fp32) {
            if (row_ok) {
#pragma unroll
              for (int q = 0; q < 4; q++) {
                if (n0 + c * 32 + q * 8 < args.N) {
                  float4* p = reinterpret_cast<float4*>(reinterpret_cast<float*>(args.D) + off + c * 32 + q * 8);
                  p[0] = make_float4(__uint_as_float(r[q * 8]), __uint_as_float(r[q * 8 + 1]), __uint_as_float(r[q * 8 + 2]), __uint_as_float(r[q * 8 + 3]));
                  p[1] = make_float4(__uint_as_float(r[q * 8 + 4]), __uint_as_float(r[q * 8 + 5]), __uint_as_float(r[q * 8 + 6]), __uint_as_float(r[q * 8 + 7]));
                }
              }
            }
          } else {
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] = __uint_as_float(r[j]);
            epi_store32_bf16(staging + (warp - 2) * kStgWarpBytes, v, row_ok, dbf + c * 32, args.N - (n0 + c * 32));
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane_id() == 0) mbar_arrive(tempty0 + 8 * buf);
        if (++buf == kAcc) { buf = 0; bphase ^= 1; }
      }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    // give copies still in flight time to land before the shared memory is handed back
    for (int i = 0; i < 2000; i++) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, kTmemCols); }
}

// ---- host side ---------------------------------------------------------------------------------
struct TmapKey {
  const void* p; uint64_t d0, d1, d2, s1, s2; uint32_t b0, b1; int dt;
  bool operator==(const TmapKey& o) const {
    return p == o.p && d0 == o.d0 && d1 == o.d1 && d2 == o.d2 && s1 == o.s1 && s2 == o.s2 && b0 == o.b0 && b1 == o.b1 && dt == o.dt;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = (size_t)k.p;
    for (uint64_t v : {k.d0, k.d1, k.d2, k.s1, k.s2, (uint64_t)k.b0, (uint64_t)k.b1, (uint64_t)k.dt}) h = h * 1000003u ^ (size_t)v;
    return h;
  }
};

// [groups][rows][K] K-major tensor -> 3-D map, box {128 bytes of K, box_rows, 1}, 128B swizzle.
static int get_tmap_kmajor(CUtensorMap* out, const void* base, bool fp8, uint64_t K, uint64_t rows, uint64_t groups,
                           uint64_t row_stride_elems, uint64_t group_stride_elems, uint32_t box_rows) {
  static std::mutex mu;
  static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  const uint64_t es = fp8 ? 1 : 2;
  TmapKey key{base, K, rows, groups, row_stride_elems * es, group_stride_elems * es, (uint32_t)(kKBytes / es), box_rows, fp8 ? TMA_U8 : TMA_BF16};
  std::lock_guard<std::mutex> lk(mu);
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return 0; }
  uint64_t dims[3] = {K, rows, groups};
  uint64_t strides[2] = {row_stride_elems * es, group_stride_elems * es};
  uint32_t box[3] = {(uint32_t)(kKBytes / es), box_rows, 1};
  if (groups > 1 && group_stride_elems < row_stride_elems) {
    // heads interleaved inside a row ([rows, groups, K] memory order): keep strides ascending, the kernel swaps coordinates
    dims[1] = groups; dims[2] = rows; strides[0] = group_stride_elems * es; strides[1] = row_stride_elems * es;
    box[1] = 1; box[2] = box_rows;
  }
  int rc = make_tmap(out, base, fp8 ? TMA_U8 : TMA_BF16, 3, dims, strides, box, TMA_SW_128);
  if (rc == 0) { if (cache.size() > 8192) cache.clear(); cache.emplace(key, *out); }
  return rc;
}

static int num_sms() {
  static int n = 0;
  if (!n) { int dev; cudaGetDevice(&dev); cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev); }
  return n;
}

template <int BLOCK_N, bool kFP8, bool kBS>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& a, int grid, cudaStream_t st) {
  auto kern = gemm_kernel<BLOCK_N, kFP8, kBS>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<BLOCK_N>::kBytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  kern<<<grid, EpiCfg<BLOCK_N, kBS>::kThreads, Smem<BLOCK_N>::kBytes, st>>>(ta, tb, a);
  return (int)cudaGetLastError();
}

}  // namespace ne

using namespace ne;

// dtype: 0 = bf16 operands, 1 = fp8 e4m3 operands with block scales (sa/sb required).
// A [groups, M, K] (row stride lda, group stride a_gs), B [groups, N, K] (contiguous), D [groups, M, N] (row stride ldd).
// masked_m: device int32 [groups] or null.  row_start: device int32 [groups] for the contiguous grouped layout (A and D
// are then flat [M, *] matrices and masked_m holds the per-group row counts) or null.
// Returns 0 or a CUDA / argument error code.
extern "C" int ne_gemm(const void* A, long long lda, long long a_gs, const void* B, void* D, long long ldd, long long d_gs,
                       int M, int N, int K, int groups, const int* masked_m, const int* row_start, int dtype, const float* sa, int sa_ld,
                       long long sa_gs, const float* sb, int out_fp32, int block_n_hint, const long long* row_dst, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || groups <= 0) return 0;
  const bool fp8 = dtype == 1;
  if (N % 8 != 0 || (K * (fp8 ? 1 : 2)) % 16 != 0 || (lda * (fp8 ? 1 : 2)) % 16 != 0) return 1001;
  if (fp8 && (K % 128 != 0 || !sa || !sb)) return 1002;
  if ((ldd * (out_fp32 ? 4 : 2)) % 16 != 0) return 1003;
  const int m_blocks = (M + kBlockM - 1) / kBlockM;
  // pick the widest N tile that still yields about one tile per SM; fp8 promotion keeps BLOCK_N accumulators in registers
  int bn = block_n_hint;
  if (bn == 0) {
    if (fp8 && !row_start && !masked_m) {
      // dense block-scaled GEMM: the serial K loop of a tile dominates at small M, so take the fewest waves of
      // tiles and, among equals, the narrowest tile (more SMs pulling weights at the same time)
      long long best_waves = 1ll << 60;
      bn = 128;
      for (int c : {128, 64, 32}) {
        long long tiles = (long long)groups * m_blocks * ((N + c - 1) / c);
        long long waves = (tiles + num_sms() - 1) / num_sms();
        if (waves <= best_waves) { best_waves = waves; bn = c; }
      }
    } else {
      const int cands[4] = {256, 128, 64, 32};
      bn = 32;
      for (int c : cands) {
        if (fp8 && c > 128) continue;
        long long tiles = (long long)groups * m_blocks * ((N + c - 1) / c);
        if (tiles >= num_sms() || c == 32) { bn = c; break; }
      }
      if (!fp8 && bn == 256 && N % 256 != 0 && N < 2048) bn = 128;
    }
  }
  if (fp8 && bn > 128) bn = 128;
  CUtensorMap ta, tb;
  if (row_start || groups == 1) a_gs = (long long)M * lda;
  int rc = get_tmap_kmajor(&ta, A, fp8, (uint64_t)K, (uint64_t)M, (uint64_t)(row_start ? 1 : groups), (uint64_t)lda, (uint64_t)a_gs, kBlockM);
  if (rc) return 2000 + rc;
  rc = get_tmap_kmajor(&tb, B, fp8, (uint64_t)K, (uint64_t)N, (uint64_t)groups, (uint64_t)K, (uint64_t)N * K, (uint32_t)bn);
  if (rc) return 3000 + rc;
  GemmArgs a;
  a.a_group_inner = (!row_start && groups > 1 && a_gs < lda) ? 1 : 0;
  a.M = M; a.N = N; a.K = K; a.groups = groups; a.masked_m = masked_m; a.row_start = row_start; a.D = D; a.ldd = ldd; a.d_group_stride = d_gs;
  if (row_start) { a.d_group_stride = 0; sa_gs = 0; if (!masked_m) return 1004; }
  a.sa = sa; a.sa_ld = sa_ld; a.sa_group_stride = sa_gs; a.sb = sb;
  a.sb_group_stride = (long long)((N + 127) / 128) * (K / 128); a.out_fp32 = out_fp32;
  a.row_dst = row_dst; a.rd_group_stride = row_start ? 0 : M;
  if (row_dst && out_fp32) return 1005;
  long long tiles = (long long)groups * m_blocks * ((N + bn - 1) / bn);
  int grid = (int)(tiles < num_sms() ? tiles : num_sms());
  if (fp8) {
    switch (bn) {
      case 128: return launch<128, true, true>(ta, tb, a, grid, stream);
      case 64: return launch<64, true, true>(ta, tb, a, grid, stream);
      default: return launch<32, true, true>(ta, tb, a, grid, stream);
    }
  }
  switch (bn) {
    case 256: return launch<256, false, false>(ta, tb, a, grid, stream);
    case 128: return launch<128, false, false>(ta, tb, a, grid, stream);
    case 64: return launch<64, false, false>(ta, tb, a, grid, stream);
    default: return launch<32, false, false>(ta, tb, a, grid, stream);
  }
}

extern "C" int ne_get_status(int* out8) {
  return (int)cudaMemcpyFromSymbol(out8, g_status, sizeof(int) * 8);
}
extern "C" int ne_clear_status() {
  int z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  return (int)cudaMemcpyToSymbol(g_status, z, sizeof(z));
}
